// Contraction entry points of the C ABI: matmul / gemm, fused linear forward+backward and the
// conv2d trio (forward, input gradient, filter gradient) as implicit GEMMs.
// f32 -> tcgen05 TF32 engine (fxb_umma_engine.cuh), f64 -> DMMA engine (fxb_dmma_engine.cuh).
#include "fxb_umma_engine.cuh"
#include "fxb_umma_tma_engine.cuh"
#include "fxb_umma_tma_wgrad.cuh"
#include "fxb_dmma_engine.cuh"
#include "fxb_small.cuh"
#include "fxb_small_umma.cuh"

#include <algorithm>

namespace fxb {

// Adds split-K partial results in split order: out[i] = sum_z part[z*stride + i].
template <typename T>
__global__ void splitk_reduce_kernel(const T* __restrict__ part, T* __restrict__ out, int64_t n, int64_t stride,
                                     int splits) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        T acc = part[i];
        for (int z = 1; z < splits; ++z) acc += part[(int64_t)z * stride + i];
        out[i] = acc;
    }
}

// The same for a split forward convolution: out[n][k][p] = act(sum_z part[z][...] + bias[k]).
__global__ void __launch_bounds__(256) splitk_bias_act_kernel(const float* __restrict__ part, float* __restrict__ out, int64_t n,
                                                              int64_t stride, int splits, const float* __restrict__ bias,
                                                              FastDiv dP, int K, int act) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float acc = part[i];
        for (int z = 1; z < splits; ++z) acc += part[(int64_t)z * stride + i];
        if (bias != nullptr) acc += __ldg(bias + dP.div((uint32_t)i) % (uint32_t)K);
        out[i] = act_apply<float>(acc, act);
    }
}

// ------------------------------------------------------------------------------------------
// Pre-split kernels of the copy-engine convolution path (f32).  They rewrite an operand once into
// TF32 "hi" (round to nearest) and exact remainder "lo" arrays whose 4-element K chunks are
// contiguous, so the contraction kernel can fill its operand tiles with 16-byte cp.async copies.
//
// Image NCHW -> channel slabs S[n][c4][p][4] (4 consecutive channels per pixel, zero padded to a
// multiple of 4 channels), or S[c4][n][p][4] with `slab_major`.  With `aux` the value is first
// multiplied by act'(aux) (dZ = dY * act'(Y)).
__global__ void __launch_bounds__(256) split_image_to_slabs_kernel(const float* __restrict__ x, const float* __restrict__ aux,
                                                                   float* __restrict__ hi, float* __restrict__ lo, int C,
                                                                   int C4, int HW, int64_t total, FastDiv dHW, FastDiv dC4,
                                                                   int act, int sig_math, int slab_major, int N) {
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        uint32_t q, p, n, c4;
        dHW.divmod((uint32_t)idx, q, p);
        dC4.divmod(q, n, c4);
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int c = (int)c4 * 4 + i;
            float t = 0.f;
            if (c < C) {
                const int64_t src = ((int64_t)n * C + c) * HW + p;
                t = __ldg(x + src);
                if (aux) t *= act_grad_factor<float>(__ldg(aux + src), act, sig_math);
            }
            v[i] = t;
        }
        uint4 h;
        h.x = cvt_tf32_rna(v[0]); h.y = cvt_tf32_rna(v[1]); h.z = cvt_tf32_rna(v[2]); h.w = cvt_tf32_rna(v[3]);
        const int64_t o = (slab_major ? ((int64_t)c4 * N + n) * HW + p : idx) * 4;
        *reinterpret_cast<uint4*>(hi + o) = h;
        *reinterpret_cast<float4*>(lo + o) =
            make_float4(v[0] - __uint_as_float(h.x), v[1] - __uint_as_float(h.y), v[2] - __uint_as_float(h.z),
                        v[3] - __uint_as_float(h.w));
    }
}

// Filter KCRS -> out[row][tap][q][4].  transpose == 0: row = k, channels c = 4q+i (forward operand);
// transpose == 1: row = c, output channels k = 4q+i (input-gradient operand).
__global__ void __launch_bounds__(256) split_filter_kernel(const float* __restrict__ w, float* __restrict__ hi,
                                                           float* __restrict__ lo, int K, int C, int RS, int Q, int rows,
                                                           int transpose) {
    const int total = rows * RS * Q;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int q = idx % Q, tap = (idx / Q) % RS, row = idx / (Q * RS);
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int inner = q * 4 + i;
            const int k = transpose ? inner : row, c = transpose ? row : inner;
            v[i] = (k < K && c < C) ? __ldg(w + ((int64_t)k * C + c) * RS + tap) : 0.f;
        }
        uint4 h;
        h.x = cvt_tf32_rna(v[0]); h.y = cvt_tf32_rna(v[1]); h.z = cvt_tf32_rna(v[2]); h.w = cvt_tf32_rna(v[3]);
        *reinterpret_cast<uint4*>(hi + (int64_t)idx * 4) = h;
        *reinterpret_cast<float4*>(lo + (int64_t)idx * 4) =
            make_float4(v[0] - __uint_as_float(h.x), v[1] - __uint_as_float(h.y), v[2] - __uint_as_float(h.z),
                        v[3] - __uint_as_float(h.w));
    }
}

// ------------------------------------------------------------------------------------------
// Pre-split kernels of the tensor-map (TMA) convolution path.
//
// Image NCHW -> class slabs S[plane][n][iy][ix][4], plane = (cy*sw + cx)*Q + q: slab q holds channels
// 4q..4q+3, class (cy, cx) holds the padded-image pixels (iy*sh + cy, ix*sw + cx); pixel (y, x) of
// the image sits at padded position (y + ph, x + pw), cells outside the image are written as zeros.
// A filter tap (r, s) of a strided convolution then reads the unit-stride window that starts at
// (oy + r/sh, ox + s/sw) of class (r%sh, s%sw).
__global__ void __launch_bounds__(256) split_image_to_class_slabs_kernel(const float* __restrict__ x, float* __restrict__ hi,
                                                                         float* __restrict__ lo, int C, int H, int W, int Q,
                                                                         int sh, int sw, int ph, int pw, int64_t total,
                                                                         FastDiv dWc, FastDiv dHc, FastDiv dN, FastDiv dQ,
                                                                         int N, int Hc, int Wc) {
    // One thread per (cy, q, n, iy, ix); it writes the cell of every x class, so that a warp reads
    // whole sectors of the image row even when the stride skips pixels.
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        uint32_t t0, ix, t1, iy, n, pq, cy, q;
        dWc.divmod((uint32_t)idx, t0, ix);
        dHc.divmod(t0, t1, iy);
        dN.divmod(t1, pq, n);
        dQ.divmod(pq, cy, q);
        const int y = (int)iy * sh + (int)cy - ph;
        const bool yin = (unsigned)y < (unsigned)H;
        for (int cx = 0; cx < sw; ++cx) {
            const int xx = (int)ix * sw + cx - pw;
            const bool in = yin && (unsigned)xx < (unsigned)W;
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int c = (int)q * 4 + i;
                v[i] = (in && c < C) ? __ldg(x + (((int64_t)n * C + c) * H + y) * W + xx) : 0.f;
            }
            uint4 h;
            h.x = cvt_tf32_rna(v[0]); h.y = cvt_tf32_rna(v[1]); h.z = cvt_tf32_rna(v[2]); h.w = cvt_tf32_rna(v[3]);
            const int plane = ((int)cy * sw + cx) * Q + (int)q;
            const int64_t o = ((((int64_t)plane * N + n) * Hc + iy) * Wc + ix) * 4;
            *reinterpret_cast<uint4*>(hi + o) = h;
            *reinterpret_cast<float4*>(lo + o) =
                make_float4(v[0] - __uint_as_float(h.x), v[1] - __uint_as_float(h.y), v[2] - __uint_as_float(h.z),
                            v[3] - __uint_as_float(h.w));
        }
    }
}

// Filter KCRS -> chunk-major F[chunk][row][4] with `rows_pad` rows per chunk (rows beyond the real
// ones are zeros).  transpose == 0 (forward): row = k, chunk = tap*Q + q holds channels 4q..4q+3.
// transpose == 1 (input gradient): row = c, the chunk holds output channels 4q..4q+3, and the taps
// are grouped by stride-residue class (r % sh, s % sw): class ci starts at chunk base[ci] and
// orders its taps (r/sh, s/sw) row-major, Q chunks per tap.
struct FilterClassBase { int base[16]; };
__global__ void __launch_bounds__(256) split_filter_chunk_major_kernel(const float* __restrict__ w, float* __restrict__ hi,
                                                                       float* __restrict__ lo, int K, int C, int R, int S, int Q,
                                                                       int rows, int rows_pad, int transpose, int sh, int sw,
                                                                       FilterClassBase fc) {
    const int total = R * S * Q * rows_pad;
    for (int idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const int row = idx % rows_pad;
        const int kc = idx / rows_pad;
        const int q = kc % Q, tap = kc / Q;
        const int r = tap / S, ss = tap % S;
        const int cy = r % sh, cx = ss % sw;
        const int Sc = (S - cx + sw - 1) / sw;
        const int chunk = fc.base[cy * sw + cx] + ((r / sh) * Sc + ss / sw) * Q + q;
        float v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int inner = q * 4 + i;
            const int k = transpose ? inner : row, c = transpose ? row : inner;
            v[i] = (row < rows && k < K && c < C) ? __ldg(w + ((int64_t)k * C + c) * (R * S) + tap) : 0.f;
        }
        uint4 h;
        h.x = cvt_tf32_rna(v[0]); h.y = cvt_tf32_rna(v[1]); h.z = cvt_tf32_rna(v[2]); h.w = cvt_tf32_rna(v[3]);
        const int64_t o = ((int64_t)chunk * rows_pad + row) * 4;
        *reinterpret_cast<uint4*>(hi + o) = h;
        *reinterpret_cast<float4*>(lo + o) =
            make_float4(v[0] - __uint_as_float(h.x), v[1] - __uint_as_float(h.y), v[2] - __uint_as_float(h.z),
                        v[3] - __uint_as_float(h.w));
    }
}

// ------------------------------------------------------------------------------------------
// Pre-pass kernels of the tensor-map filter-gradient path (and, fused, of the input-gradient path).
//
// dZ = dY * act'(Y), NCHW -> DZN[g][p][o][4] (hi and lo): the values of images 4g..4g+3 at pixel p and
// output channel o, rows padded with zeros to `Kp` channels, images beyond N are zeros.  With `slab_hi`
// the same pass also writes the channel slabs S[o/4][n][p][4] that the input-gradient kernel reads, and
// with `dbpart` the bias gradient, deterministically: block (bx, by, g) adds its 4 x 32 values of each of its
// 32 output channels and writes dbpart[g * gridDim.x + bx][o]; partial_rows_sum_kernel adds the rows in order.
// Block = 4 images x 32 channels x 32 pixels through shared memory: reads coalesced along the pixels,
// writes coalesced along the channels (DZN) and along the pixels (slabs).

// ------------------------------------------------------------------------------------------
// Operand passes of the tensor-map GEMM: a matrix op(X)[rows][K] -> chunk-major F[K/4][rows_pad][4]
// (hi and lo), rows beyond `rows` and K beyond the matrix are zeros.  With `aux` (same shape and
// leading dimension) the value is first multiplied by act'(aux).
//
// K contiguous in memory (op(X) = X[rows][ld]): a block moves 32 rows x 32 chunks through shared
// memory: 16-byte loads along K, 16-byte stores along the rows.
__global__ void __launch_bounds__(256) split_matrix_kmajor_kernel(const float* __restrict__ x, const float* __restrict__ aux,
                                                                  int64_t ld, int rows, int K, int K4, int rows_pad,
                                                                  float* __restrict__ hi, float* __restrict__ lo, int vec_ok,
                                                                  int act, int sig_math) {
    __shared__ float4 tile[32][33];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int r0 = blockIdx.x * 32, q0 = blockIdx.y * 32;
    float4 v[4], a[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r0 + w * 4 + i, q = q0 + lane;
        v[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        a[i] = v[i];
        if (r < rows && q < K4) {
            const int64_t o = (int64_t)r * ld + (int64_t)q * 4;
            if (vec_ok && q * 4 + 3 < K) {
                v[i] = __ldg(reinterpret_cast<const float4*>(x + o));
                if (aux) a[i] = __ldg(reinterpret_cast<const float4*>(aux + o));
            } else {
                float t[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (q * 4 + j < K) {
                        t[j] = __ldg(x + o + j);
                        if (aux) u[j] = __ldg(aux + o + j);
                    }
                v[i] = make_float4(t[0], t[1], t[2], t[3]);
                a[i] = make_float4(u[0], u[1], u[2], u[3]);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (aux) {
            v[i].x *= act_grad_factor<float>(a[i].x, act, sig_math);
            v[i].y *= act_grad_factor<float>(a[i].y, act, sig_math);
            v[i].z *= act_grad_factor<float>(a[i].z, act, sig_math);
            v[i].w *= act_grad_factor<float>(a[i].w, act, sig_math);
            // (values outside the matrix were loaded as zeros and stay zeros: 0 * finite factor)
        }
        tile[w * 4 + i][lane] = v[i];
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int q = q0 + w * 4 + i, r = r0 + lane;
        if (q < K4 && r < rows_pad) {
            const float4 t = tile[lane][w * 4 + i];
            store_split4(hi, lo, ((int64_t)q * rows_pad + r) * 4, t.x, t.y, t.z, t.w);
        }
    }
}
// Rows contiguous in memory (op(X)(r, k) = X[k * ld + r]): one thread per (chunk, row), loads and stores
// coalesced along the rows.
__global__ void __launch_bounds__(256) split_matrix_rowmajor_kernel(const float* __restrict__ x, const float* __restrict__ aux,
                                                                    int64_t ld, int rows, int K, int rows_pad, int64_t total,
                                                                    float* __restrict__ hi, float* __restrict__ lo, int act,
                                                                    int sig_math) {
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int64_t q = idx / rows_pad;
        const int r = (int)(idx - q * rows_pad);
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int64_t k = q * 4 + j;
            float t = 0.f;
            if (r < rows && k < K) {
                t = __ldg(x + k * ld + r);
                if (aux) t *= act_grad_factor<float>(__ldg(aux + k * ld + r), act, sig_math);
            }
            v[j] = t;
        }
        store_split4(hi, lo, idx * 4, v[0], v[1], v[2], v[3]);
    }
}

__global__ void __launch_bounds__(256) pack_dz_kernel(const float* __restrict__ dy, const float* __restrict__ yact,
                                                      float* __restrict__ dzn_hi, float* __restrict__ dzn_lo,
                                                      float* __restrict__ slab_hi, float* __restrict__ slab_lo,
                                                      float* __restrict__ dbpart, int N, int K, int Kp, int P, int act,
                                                      int sig_math) {
    __shared__ float t[4][32][33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p0 = blockIdx.x * 32, o0 = blockIdx.y * 32, g = blockIdx.z;
    // all loads are issued before the first value is used (up to 32 independent loads in flight per thread)
    float vd[16], vy[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int q = warp + 8 * j;
        const int n4 = q >> 5, ol = q & 31;
        const int n = 4 * g + n4, o = o0 + ol, p = p0 + lane;
        const bool in = n < N && o < K && p < P;
        const int64_t src = ((int64_t)n * K + o) * P + p;
        vd[j] = in ? __ldg(dy + src) : 0.f;
        vy[j] = (in && yact != nullptr) ? __ldg(yact + src) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        const int q = warp + 8 * j;
        float v = vd[j];
        if (yact) v *= act_grad_factor<float>(vy[j], act, sig_math);
        t[q >> 5][q & 31][lane] = v;
    }
    __syncthreads();
    if (dbpart != nullptr && warp == 0 && o0 + lane < K) {
        float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
        for (int p = 0; p < 32; ++p) {
            s0 += t[0][lane][p]; s1 += t[1][lane][p]; s2 += t[2][lane][p]; s3 += t[3][lane][p];
        }
        dbpart[((int64_t)g * gridDim.x + blockIdx.x) * K + o0 + lane] = (s0 + s1) + (s2 + s3);
    }
    for (int i = threadIdx.x; i < 1024; i += 256) {
        const int ol = i & 31, pl = i >> 5;
        const int o = o0 + ol, p = p0 + pl;
        if (o < Kp && p < P)
            store_split4(dzn_hi, dzn_lo, (((int64_t)g * P + p) * Kp + o) * 4, t[0][ol][pl], t[1][ol][pl], t[2][ol][pl], t[3][ol][pl]);
    }
    if (slab_hi != nullptr) {
        const int K4 = (K + 3) >> 2;
        for (int i = threadIdx.x; i < 1024; i += 256) {
            const int pl = i & 31, rest = i >> 5;
            const int n4 = rest >> 3, q = rest & 7;
            const int n = 4 * g + n4, p = p0 + pl, k4 = (o0 >> 2) + q;
            if (n < N && p < P && k4 < K4)
                store_split4(slab_hi, slab_lo, (((int64_t)k4 * N + n) * P + p) * 4, t[n4][4 * q][pl], t[n4][4 * q + 1][pl],
                             t[n4][4 * q + 2][pl], t[n4][4 * q + 3][pl]);
        }
    }
}

// X NCHW -> XN[cls][g][iy][ix][c][4] (hi and lo): in padded coordinates (yp, xp) = (y + ph, x + pw), class
// cls = (yp % sh) * sw + xp % sw, cell (iy, ix) = (yp / sh, xp / sw); the four values are images 4g..4g+3,
// `Cp` channels per cell (zeros beyond C, outside the image and beyond N).
// Block = 4 images x 64 channels x a band of RY padded rows, walked in chunks of 32 cells through shared
// memory: reads coalesced along x; writes ordered by destination address (the cells of a chunk sorted by
// class, 64 channels = 1 KB per cell), so that a block emits runs of many KB instead of scattered pieces.
constexpr int XN_CT = 64;  // channels per block
__global__ void __launch_bounds__(256, 4) pack_xn_kernel(const float* __restrict__ x, float* __restrict__ xn_hi,
                                                      float* __restrict__ xn_lo, int N, int C, int Cp, int H, int W, int ph,
                                                      int pw, int Hc, int Wc, int N4, int RY, FastDiv dWp, FastDiv dsh,
                                                      FastDiv dsw) {
    __shared__ float t[4][XN_CT][33];
    __shared__ long long cell_off[32];   // XN float offset of the cell's channel 0, in destination order; -1 = no cell
    __shared__ int cell_src[32];         // which cell of the chunk that is
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int c0 = blockIdx.x * XN_CT, g = blockIdx.z;
    const int sh = (int)dsh.d, sw = (int)dsw.d;
    const int Wp = Wc * sw, Hp = Hc * sh;
    const int yp0 = blockIdx.y * RY;
    const int rows = min(RY, Hp - yp0);
    const int cells = rows * Wp;
    for (int e0 = 0; e0 < cells; e0 += 32) {
        const int e = e0 + lane;
        uint32_t ry = 0, xp = 0;
        if (e < cells) dWp.divmod((uint32_t)e, ry, xp);
        const int y = yp0 + (int)ry - ph, xx = (int)xp - pw;
        const bool in = e < cells && (unsigned)y < (unsigned)H && (unsigned)xx < (unsigned)W;
        // all loads of the chunk are issued before the first value is used (32 independent loads in flight per thread)
        float v[4 * XN_CT / 8];
#pragma unroll
        for (int j = 0; j < 4 * XN_CT / 8; ++j) {
            const int q = warp + 8 * j;
            const int n4 = q / XN_CT, cl = q - n4 * XN_CT;
            const int n = 4 * g + n4, c = c0 + cl;
            v[j] = (in && n < N && c < C) ? __ldg(x + (((int64_t)n * C + c) * H + y) * W + xx) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < 4 * XN_CT / 8; ++j) {
            const int q = warp + 8 * j;
            const int n4 = q / XN_CT, cl = q - n4 * XN_CT;
            t[n4][cl][lane] = v[j];
        }
        if (warp == 0) {
            // destination order: cells sorted by (class, position), i.e. by address
            uint32_t iy = 0, cy = 0, ix = 0, cx = 0;
            dsh.divmod((uint32_t)yp0 + ry, iy, cy);
            dsw.divmod(xp, ix, cx);
            const int cls = e < cells ? (int)cy * sw + (int)cx : sh * sw;  // cells beyond the band sort last
            int pos = 0;
            for (int v = 0; v <= sh * sw; ++v) {
                const unsigned m = __ballot_sync(0xffffffffu, cls == v);
                if (v < cls) pos += __popc(m);
                else if (v == cls) pos += __popc(m & ((1u << lane) - 1u));
            }
            cell_src[pos] = lane;
            cell_off[pos] = e < cells ? ((((long long)cls * N4 + g) * Hc + iy) * Wc + ix) * Cp * 4 : -1;
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 32 * XN_CT; i += 256) {
            const int pos = i / XN_CT, cl = i - pos * XN_CT;
            const long long off = cell_off[pos];
            const int c = c0 + cl;
            if (off >= 0 && c < Cp) {
                const int el = cell_src[pos];
                store_split4(xn_hi, xn_lo, off + (long long)c * 4, t[0][cl][el], t[1][cl][el], t[2][cl][el], t[3][cl][el]);
            }
        }
        __syncthreads();
    }
}

// out[o] = sum over b of part[b][o], b in a fixed order: block = 8 outputs x 32 row lanes, every lane keeps four
// interleaved running sums (four independent loads in flight), combined as a fixed tree, so the result does
// not depend on scheduling.
__global__ void __launch_bounds__(256) partial_rows_sum_kernel(const float* __restrict__ part, float* __restrict__ out, int K,
                                                               int rows) {
    __shared__ float red[32][9];
    const int ol = threadIdx.x & 7, bl = threadIdx.x >> 3;
    const int o = blockIdx.x * 8 + ol;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (o < K) {
        int b = bl;
        for (; b + 96 < rows; b += 128) {
            a0 += __ldg(part + (int64_t)b * K + o);
            a1 += __ldg(part + (int64_t)(b + 32) * K + o);
            a2 += __ldg(part + (int64_t)(b + 64) * K + o);
            a3 += __ldg(part + (int64_t)(b + 96) * K + o);
        }
        for (; b < rows; b += 32) a0 += __ldg(part + (int64_t)b * K + o);
    }
    red[bl][ol] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    if (bl == 0 && o < K) {
        float s[4] = {0.f, 0.f, 0.f, 0.f};
        for (int w = 0; w < 32; w += 4) {
            s[0] += red[w][ol]; s[1] += red[w + 1][ol]; s[2] += red[w + 2][ol]; s[3] += red[w + 3][ol];
        }
        out[o] = (s[0] + s[1]) + (s[2] + s[3]);
    }
}

template <typename T>
struct Problem {
    int M = 0, N = 0, K = 0;
    T* rowsum_a = nullptr;  // length M, sum over k of A(m,k)
    T* rowsum_b = nullptr;  // length N, sum over k of B(n,k)
    void* ws = nullptr;
    size_t ws_bytes = 0;
    bool allow_split = false;  // output contiguous, no bias / activation
    int64_t out_elems = 0;
};

static int pick_splits(const Context* c, int tiles, int kblocks, int min_kblocks_per_split) {
    if (tiles >= c->sm_count || kblocks < 2 * min_kblocks_per_split) return 1;
    int s = c->sm_count / tiles;
    s = std::min(s, kblocks / min_kblocks_per_split);
    return std::max(s, 1);
}

template <typename T>
static size_t split_workspace_bytes(int splits, int64_t out_elems, int ra, int rb) {
    return splits > 1 ? (size_t)splits * (size_t)(out_elems + ra + rb) * sizeof(T) : 0;
}

template <typename T>
static int finish_split(Context* c, const Problem<T>& p, T* out, int splits, cudaStream_t st) {
    T* part = static_cast<T*>(p.ws);
    const int threads = 256;
    auto blocks = [&](int64_t n) { return (int)std::min<int64_t>((n + threads - 1) / threads, (int64_t)c->sm_count * 8); };
    splitk_reduce_kernel<T><<<blocks(p.out_elems), threads, 0, st>>>(part, out, p.out_elems, p.out_elems, splits);
    T* rs = part + (size_t)splits * p.out_elems;
    if (p.rowsum_a) {
        splitk_reduce_kernel<T><<<blocks(p.M), threads, 0, st>>>(rs, p.rowsum_a, p.M, p.M, splits);
        rs += (size_t)splits * p.M;
    }
    if (p.rowsum_b) splitk_reduce_kernel<T><<<blocks(p.N), threads, 0, st>>>(rs, p.rowsum_b, p.N, p.N, splits);
    return launch_status(c, "splitk_reduce", 1 + (p.rowsum_a ? 1 : 0) + (p.rowsum_b ? 1 : 0));
}

// ------------------------------------------------------------------------------ f32 launcher
template <class LA, class LB, int BN>
static int launch_umma_bn(Context* c, const LA& la, const LB& lb, OutputWriter<float> ow, const Problem<float>& p,
                          cudaStream_t st) {
    using Cfg = UmmaCfg<BN>;
    auto kern = umma_contract_kernel<LA, LB, BN>;
    static bool attr_set[64] = {};
    if (!attr_set[c->device & 63]) {
        FXB_CUDA_OK(c, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[c->device & 63] = true;
    }
    const int tm = (p.M + UMMA_BM - 1) / UMMA_BM, tn = (p.N + BN - 1) / BN;
    const int kstages = (p.K + UMMA_BK - 1) / UMMA_BK;
    int splits = 1;
    if (p.allow_split && p.ws != nullptr) {
        splits = pick_splits(c, tm * tn, kstages, 16);
        while (splits > 1 && split_workspace_bytes<float>(splits, p.out_elems, p.rowsum_a ? p.M : 0,
                                                          p.rowsum_b ? p.N : 0) > p.ws_bytes)
            --splits;
    }
    UmmaShape shp;
    shp.M = p.M; shp.N = p.N; shp.K = p.K;
    shp.tm = tm; shp.tn = tn;
    shp.stages_per_split = std::max(1, (kstages + splits - 1) / splits);
    splits = std::max(1, (kstages + shp.stages_per_split - 1) / shp.stages_per_split);
    shp.splits = splits;
    shp.three_pass = c->math_mode == FXB_MATH_3XTF32 ? 1 : 0;
    float* final_out = ow.out;
    float* rsa = p.rowsum_a;
    float* rsb = p.rowsum_b;
    if (splits > 1) {
        float* part = static_cast<float*>(p.ws);
        ow.out = part;
        ow.split_stride = p.out_elems;
        float* rs = part + (size_t)splits * p.out_elems;
        if (rsa) { rsa = rs; rs += (size_t)splits * p.M; }
        if (rsb) rsb = rs;
    }
    const long long items = (long long)tm * tn * splits;
    const int grid = (int)std::min<long long>(items, c->sm_count);  // persistent: one CTA per SM
    kern<<<grid, UMMA_THREADS, Cfg::SMEM_BYTES, st>>>(la, lb, ow, shp, rsa, rsb, c->d_status);
    int rc = launch_status(c, "umma_contract_kernel");
    if (rc != FXB_OK) return rc;
    if (splits > 1) return finish_split<float>(c, p, final_out, splits, st);
    return FXB_OK;
}

template <class LA, class LB>
static int launch_contract(Context* c, const LA& la, const LB& lb, const OutputWriter<float>& ow,
                           const Problem<float>& p, cudaStream_t st) {
    if (p.N <= 16) return launch_umma_bn<LA, LB, 16>(c, la, lb, ow, p, st);
    if (p.N <= 64) return launch_umma_bn<LA, LB, 64>(c, la, lb, ow, p, st);
    return launch_umma_bn<LA, LB, 128>(c, la, lb, ow, p, st);
}

// ------------------------------------------------------------------------------ f64 launcher
template <class LA, class LB, int BN>
static int launch_dmma_bn(Context* c, const LA& la, const LB& lb, OutputWriter<double> ow, const Problem<double>& p,
                          cudaStream_t st) {
    using Cfg = DmmaCfg<BN>;
    auto kern = dmma_contract_kernel<LA, LB, BN>;
    static bool attr_set[64] = {};
    if (!attr_set[c->device & 63]) {
        FXB_CUDA_OK(c, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[c->device & 63] = true;
    }
    const int tm = (p.M + DMMA_BM - 1) / DMMA_BM, tn = (p.N + BN - 1) / BN;
    const int ktiles = (p.K + DMMA_BK - 1) / DMMA_BK;
    int splits = 1;
    if (p.allow_split && p.ws != nullptr) {
        splits = pick_splits(c, tm * tn, ktiles, 16);
        while (splits > 1 && split_workspace_bytes<double>(splits, p.out_elems, p.rowsum_a ? p.M : 0,
                                                           p.rowsum_b ? p.N : 0) > p.ws_bytes)
            --splits;
    }
    DmmaShape shp;
    shp.M = p.M; shp.N = p.N; shp.K = p.K;
    shp.ktiles_per_split = std::max(1, (ktiles + splits - 1) / splits);
    splits = std::max(1, (ktiles + shp.ktiles_per_split - 1) / shp.ktiles_per_split);
    double* final_out = ow.out;
    double* rsa = p.rowsum_a;
    double* rsb = p.rowsum_b;
    if (splits > 1) {
        double* part = static_cast<double*>(p.ws);
        ow.out = part;
        ow.split_stride = p.out_elems;
        double* rs = part + (size_t)splits * p.out_elems;
        if (rsa) { rsa = rs; rs += (size_t)splits * p.M; }
        if (rsb) rsb = rs;
    }
    if (tn > 65535 || splits > 65535)
        return fail(c, FXB_ERR_UNSUPPORTED, "f64 contraction: more than 65535 column tiles (N > 4 million) is not supported");
    dim3 grid(tm, tn, splits);
    kern<<<grid, DMMA_THREADS, Cfg::SMEM_BYTES, st>>>(la, lb, ow, shp, rsa, rsb);
    int rc = launch_status(c, "dmma_contract_kernel");
    if (rc != FXB_OK) return rc;
    if (splits > 1) return finish_split<double>(c, p, final_out, splits, st);
    return FXB_OK;
}

template <class LA, class LB>
static int launch_contract(Context* c, const LA& la, const LB& lb, const OutputWriter<double>& ow,
                           const Problem<double>& p, cudaStream_t st) {
    if (p.N <= 64) return launch_dmma_bn<LA, LB, 64>(c, la, lb, ow, p, st);
    return launch_dmma_bn<LA, LB, 128>(c, la, lb, ow, p, st);
}

// Upper bound on what any split decision may ask for (used by the *_workspace_bytes queries).
static size_t split_ws_upper(const Context* c, int64_t M, int64_t N, int64_t K, int64_t out_elems, int ra, int rb,
                             size_t elem) {
    // the f64 engine has the smaller tiles => the larger split counts
    const int tile_n = elem == 8 ? (N <= 64 ? 64 : 128) : (N <= 16 ? 16 : N <= 64 ? 64 : 128);
    const int tm = (int)((M + 127) / 128), tn = (int)((N + tile_n - 1) / tile_n);
    const int kunit = elem == 8 ? DMMA_BK : UMMA_BK;
    const int minper = 16;
    const int ku = (int)((K + kunit - 1) / kunit);
    const int splits = pick_splits(c, tm * tn, ku, minper);
    return splits > 1 ? (size_t)splits * (size_t)(out_elems + ra + rb) * elem : 0;
}

// ------------------------------------------------------------------------------ helpers
template <typename T>
static bool aligned16(const T* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

template <typename T, bool KC>
static DenseLoader<T, KC> make_dense(const Context* c, const T* p, int64_t ld, int rows, int K, const T* aux, int act) {
    DenseLoader<T, KC> l;
    l.p = p; l.aux = aux; l.ld = ld; l.rows = rows; l.K = K;
    l.act = aux ? act : FXB_ACT_NONE;
    l.sig_math = c->sigmoid_grad_math;
    const int vec = sizeof(T) == 4 ? 4 : 2;
    l.vec_ok = KC && aligned16(p) && (aux == nullptr || aligned16(aux)) && (ld % vec == 0);
    return l;
}

template <typename T>
static OutputWriter<T> make_rowmajor_writer(T* out, int64_t ldm, const T* bias, int act, int M, int N) {
    OutputWriter<T> w;
    w.out = out; w.bias = bias; w.ldm = ldm; w.plane = 0; w.img_stride = 0; w.nstr = 1; w.dplane.init(1);
    w.gw = 0; w.dgw.init(1); w.goff = w.gys = w.gxs = 0;
    w.act = act; w.M = M; w.N = N; w.split_stride = 0;
    return w;
}
template <typename T>
static OutputWriter<T> make_plane_writer(T* out, int plane, int64_t img_stride, const T* bias, int act, int M, int N) {
    OutputWriter<T> w;
    w.out = out; w.bias = bias; w.ldm = 0; w.plane = plane; w.img_stride = img_stride; w.nstr = plane; w.dplane.init(plane);
    w.gw = 0; w.dgw.init(1); w.goff = w.gys = w.gxs = 0;
    w.act = act; w.M = M; w.N = N; w.split_stride = 0;
    return w;
}

static bool fits_i32(int64_t v) { return v >= 0 && v < (int64_t)1 << 31; }

// GEMM on the tensor-map convolution engine (defined with that engine's host code below).
static bool tma_gemm_wanted(const Context* c, int64_t M, int64_t N, int64_t K);
static size_t tma_gemm_bytes(int64_t M, int64_t N, int64_t K);
static int gemm_tma(Context* c, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
                    int64_t ldb, float* C, int64_t ldc, const float* bias, int act, const float* a_aux, int a_act, void* ws,
                    cudaStream_t st, bool* used);

template <typename T>
static int gemm_impl(Context* c, int ta, int tb, int64_t M, int64_t N, int64_t K, const T* A, int64_t lda, const T* B,
                     int64_t ldb, T* C, int64_t ldc, const T* bias, int act, const T* a_aux, int a_act, T* rowsum_a,
                     void* ws, size_t ws_bytes, cudaStream_t st) {
    FXB_CHECK_ARG(c, M >= 0 && N >= 0 && K >= 0, "Matrix multiplication requires non-negative sizes");
    FXB_CHECK_ARG(c, fits_i32(M) && fits_i32(N) && fits_i32(K) && fits_i32(M * 1) , "Matrix dimensions exceed 2^31-1");
    if (M == 0 || N == 0) return FXB_OK;
    FXB_CHECK_ARG(c, A && B && C, "Matrix multiplication got a null buffer");
    FXB_CHECK_ARG(c, lda >= (ta ? M : K) && ldb >= (tb ? K : N) && ldc >= N, "Leading dimension smaller than the row length");
    FXB_CHECK_ARG(c, act >= FXB_ACT_NONE && act <= FXB_ACT_TANH, "Unknown activation code");
    if constexpr (sizeof(T) == 4) {
        // Large products with a workspace: operands pre-split once, tiles fed by the copy engine.
        if (c->operand_path == FXB_PATH_AUTO && rowsum_a == nullptr && ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255) == 0 &&
            tma_gemm_wanted(c, M, N, K) && ws_bytes >= tma_gemm_bytes(M, N, K)) {
            bool used = false;
            const int rc = gemm_tma(c, ta, tb, M, N, K, A, lda, B, ldb, C, ldc, bias, act, a_aux, a_act, ws, st, &used);
            if (rc || used) return rc;
        }
    }
    Problem<T> p;
    p.M = (int)M; p.N = (int)N; p.K = (int)K;
    p.rowsum_a = rowsum_a;
    p.ws = ws; p.ws_bytes = ws_bytes;
    p.allow_split = (bias == nullptr && act == FXB_ACT_NONE && ldc == N);
    p.out_elems = M * N;
    auto ow = make_rowmajor_writer<T>(C, ldc, bias, act, (int)M, (int)N);
    if (!ta && tb)
        return launch_contract(c, make_dense<T, true>(c, A, lda, p.M, p.K, a_aux, a_act),
                               make_dense<T, true>(c, B, ldb, p.N, p.K, nullptr, 0), ow, p, st);
    if (!ta && !tb)
        return launch_contract(c, make_dense<T, true>(c, A, lda, p.M, p.K, a_aux, a_act),
                               make_dense<T, false>(c, B, ldb, p.N, p.K, nullptr, 0), ow, p, st);
    if (ta && tb)
        return launch_contract(c, make_dense<T, false>(c, A, lda, p.M, p.K, a_aux, a_act),
                               make_dense<T, true>(c, B, ldb, p.N, p.K, nullptr, 0), ow, p, st);
    return launch_contract(c, make_dense<T, false>(c, A, lda, p.M, p.K, a_aux, a_act),
                           make_dense<T, false>(c, B, ldb, p.N, p.K, nullptr, 0), ow, p, st);
}

static int make_geom(Context* c, const fxb_conv2d_desc* d, ConvGeom& g) {
    FXB_CHECK_ARG(c, d != nullptr, "Conv2D descriptor is null");
    FXB_CHECK_ARG(c, d->N > 0 && d->C > 0 && d->H > 0 && d->W > 0 && d->K > 0 && d->R > 0 && d->S > 0,
                  "Conv2D requires 4D tensors [batch, channels, height, width] with positive sizes");
    FXB_CHECK_ARG(c, d->stride_h > 0 && d->stride_w > 0 && d->pad_h >= 0 && d->pad_w >= 0,
                  "Conv2D stride must be positive and padding non-negative");
    FXB_CHECK_ARG(c, d->H + 2 * d->pad_h >= d->R && d->W + 2 * d->pad_w >= d->S,
                  "Conv2D filter larger than the padded input");
    if (d->R > 32 || d->S > 32) return fail(c, FXB_ERR_UNSUPPORTED, "Conv2D filters larger than 32x32 are not supported");
    const int64_t OH = (d->H + 2 * d->pad_h - d->R) / d->stride_h + 1;
    const int64_t OW = (d->W + 2 * d->pad_w - d->S) / d->stride_w + 1;
    FXB_CHECK_ARG(c, fits_i32(d->N * d->C * d->H * d->W) && fits_i32(d->N * d->K * OH * OW) &&
                         fits_i32(d->K * d->C * d->R * d->S) && fits_i32(d->N * OH * OW) && fits_i32(d->N * d->H * d->W),
                  "Conv2D tensor has more than 2^31-1 elements");
    g.N = (int)d->N; g.C = (int)d->C; g.H = (int)d->H; g.W = (int)d->W; g.K = (int)d->K; g.R = (int)d->R; g.S = (int)d->S;
    g.OH = (int)OH; g.OW = (int)OW; g.sh = (int)d->stride_h; g.sw = (int)d->stride_w; g.ph = (int)d->pad_h; g.pw = (int)d->pad_w;
    g.finish();
    return FXB_OK;
}

// ---- copy-engine convolution path (f32, needs a workspace for the pre-split operands) --------
static size_t align_up256(size_t v) { return (v + 255) & ~(size_t)255; }

struct SplitWs {
    float *a_hi, *a_lo, *b_hi, *b_lo;
    size_t bytes;
};
// Carves [image hi | image lo | filter hi | filter lo] out of a workspace.
static SplitWs carve_split_ws(void* ws, int64_t image_floats, int64_t filter_floats) {
    SplitWs r;
    char* p = static_cast<char*>(ws);
    const size_t ia = align_up256((size_t)image_floats * 4), fa = align_up256((size_t)filter_floats * 4);
    r.a_hi = reinterpret_cast<float*>(p);
    r.a_lo = reinterpret_cast<float*>(p + ia);
    r.b_hi = reinterpret_cast<float*>(p + 2 * ia);
    r.b_lo = reinterpret_cast<float*>(p + 2 * ia + fa);
    r.bytes = 2 * ia + 2 * fa;
    return r;
}
// ---- tensor-map (TMA) convolution path: geometry shared by the size queries and the launches ----
static int tile_cols(int n) { return n <= 16 ? 16 : n <= 64 ? 64 : 128; }
static int round_up(int v, int m) { return (v + m - 1) / m * m; }
static int log2_ceil(int v) { int l = 0; while ((1 << l) < v) ++l; return l; }

// An M tile is a TW x TH patch of the row grid in NI consecutive images, TW*TH*NI = 128.
struct PatchPlan { int tw_log, th_log, ni, PW, PH; };
static PatchPlan plan_patch(int Hv, int Wv) {
    PatchPlan p;
    p.tw_log = std::min(4, log2_ceil(Wv));
    p.th_log = std::min(7 - p.tw_log, log2_ceil(Hv));
    p.ni = 128 >> (p.tw_log + p.th_log);
    p.PW = (Wv + (1 << p.tw_log) - 1) >> p.tw_log;
    p.PH = (Hv + (1 << p.th_log) - 1) >> p.th_log;
    return p;
}
struct TmaFpropLayout {
    int Q, planes, Hc, Wc, rows_pad;
    int64_t image_floats, filter_floats;
};
static TmaFpropLayout tma_fprop_layout(const ConvGeom& g) {
    TmaFpropLayout l;
    l.Q = (g.C + 3) / 4;
    l.planes = g.sh * g.sw * l.Q;
    l.Hc = (g.H - 1 + g.ph) / g.sh + 1;
    l.Wc = (g.W - 1 + g.pw) / g.sw + 1;
    l.rows_pad = round_up(g.K, tile_cols(g.K));
    l.image_floats = (int64_t)g.N * l.planes * l.Hc * l.Wc * 4;
    l.filter_floats = (int64_t)g.RS * l.Q * l.rows_pad * 4;
    return l;
}
static bool tma_stride_ok(const ConvGeom& g) { return g.sh * g.sw <= 16; }

// Split-K plan of the tensor-map forward convolution: with fewer tiles than half the SMs, the K stages of a
// tile are divided among several CTAs (partial sums in the workspace, added in split order afterwards).
struct FpropSplit { int splits, stages_per_split; };
static FpropSplit fprop_split_plan(const Context* c, const ConvGeom& g) {
    const PatchPlan pp = plan_patch(g.OH, g.OW);
    const int bn = tile_cols(g.K);
    const int tiles = (g.N + pp.ni - 1) / pp.ni * pp.PH * pp.PW * ((g.K + bn - 1) / bn);
    const int stages = (g.RS * ((g.C + 3) / 4) + TMA_KCH - 1) / TMA_KCH;
    FpropSplit f{1, stages};
    if (tiles * 2 > c->sm_count || stages < 8) return f;
    const int want = std::max(1, std::min(c->sm_count / tiles, stages / 4));
    f.stages_per_split = (stages + want - 1) / want;
    f.splits = (stages + f.stages_per_split - 1) / f.stages_per_split;
    return f;
}
static size_t fprop_split_bytes(const Context* c, const ConvGeom& g) {
    const int64_t C4 = (g.C + 3) / 4;
    size_t need = carve_split_ws(nullptr, (int64_t)g.N * C4 * g.HW * 4, (int64_t)g.K * g.RS * C4 * 4).bytes;
    if (tma_stride_ok(g)) {
        const TmaFpropLayout l = tma_fprop_layout(g);
        const FpropSplit f = fprop_split_plan(c, g);
        const size_t part = f.splits > 1 ? align_up256((size_t)f.splits * g.N * g.K * g.P * 4) : 0;
        need = std::max(need, align_up256(carve_split_ws(nullptr, l.image_floats, l.filter_floats).bytes) + part);
    }
    return need;
}
static size_t dgrad_split_bytes(const ConvGeom& g) {
    const int64_t K4 = (g.K + 3) / 4;
    const int64_t rows_pad = round_up(g.C, tile_cols(g.C));
    return carve_split_ws(nullptr, (int64_t)g.N * K4 * g.P * 4, std::max<int64_t>(g.C, rows_pad) * g.RS * K4 * 4).bytes;
}

static int launch_split_image(Context* c, const float* x, const float* aux, float* hi, float* lo, int N, int C, int HW,
                              int act, cudaStream_t st, bool slab_major = false) {
    const int C4 = (C + 3) / 4;
    const int64_t total = (int64_t)N * C4 * HW;
    if (total >= ((int64_t)1 << 31)) return fail(c, FXB_ERR_UNSUPPORTED, "Conv2D tensor too large for the pre-split path");
    const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)c->sm_count * 16);
    split_image_to_slabs_kernel<<<blocks, 256, 0, st>>>(x, aux, hi, lo, C, C4, HW, total, FastDiv((uint32_t)HW),
                                                        FastDiv((uint32_t)C4), aux ? act : FXB_ACT_NONE, c->sigmoid_grad_math,
                                                        slab_major ? 1 : 0, N);
    return launch_status(c, "split_image_to_slabs_kernel");
}
static int launch_split_filter(Context* c, const float* w, float* hi, float* lo, int K, int C, int RS, bool transpose,
                               cudaStream_t st) {
    const int Q = transpose ? (K + 3) / 4 : (C + 3) / 4, rows = transpose ? C : K;
    const int total = rows * RS * Q;
    const int blocks = std::max(1, std::min((total + 255) / 256, c->sm_count * 8));
    split_filter_kernel<<<blocks, 256, 0, st>>>(w, hi, lo, K, C, RS, Q, rows, transpose ? 1 : 0);
    return launch_status(c, "split_filter_kernel");
}

template <int BN, bool VEC>
static int launch_tma_bn(Context* c, const TmaConvParams& prm, cudaStream_t st) {
    using Cfg = TmaCfg<BN>;
    auto kern = umma_tma_conv_kernel<BN, VEC>;
    static bool attr_set[64] = {};
    if (!attr_set[c->device & 63]) {
        FXB_CUDA_OK(c, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[c->device & 63] = true;
    }
    const long long items = (long long)prm.tm * prm.tn * prm.ncls * prm.splits;
    const int grid = (int)std::min<long long>(items, c->sm_count);  // persistent: one CTA per SM
    kern<<<grid, TMA_CONV_THREADS, Cfg::SMEM_BYTES, st>>>(prm, c->d_status);
    return launch_status(c, "umma_tma_conv_kernel");
}
static int launch_tma(Context* c, const TmaConvParams& prm, int bn, cudaStream_t st) {
    if (prm.vec_store) {
        if (bn == 16) return launch_tma_bn<16, true>(c, prm, st);
        if (bn == 64) return launch_tma_bn<64, true>(c, prm, st);
        return launch_tma_bn<128, true>(c, prm, st);
    }
    if (bn == 16) return launch_tma_bn<16, false>(c, prm, st);
    if (bn == 64) return launch_tma_bn<64, false>(c, prm, st);
    return launch_tma_bn<128, false>(c, prm, st);
}

// Tensor maps of one slab image (hi and lo): dims [Ws*4, Hs, N, planes]; box = one patch of `chunks`
// consecutive planes (8 when the slabs per tap are a multiple of 8, so that a stage never straddles taps).
static bool encode_slab_maps(TmaConvParams& prm, const float* hi, const float* lo, int Ws, int Hs, int planes, int N,
                             const PatchPlan& pp, int slabs_per_tap) {
    prm.a_chunks = slabs_per_tap % TMA_KCH == 0 ? TMA_KCH : 1;
    const uint64_t dims[4] = {(uint64_t)Ws * 4, (uint64_t)Hs, (uint64_t)N, (uint64_t)planes};
    const uint64_t str[3] = {(uint64_t)Ws * 16, (uint64_t)Hs * Ws * 16, (uint64_t)N * Hs * Ws * 16};
    const uint32_t box[4] = {(uint32_t)(4 << pp.tw_log), (uint32_t)(1 << pp.th_log), (uint32_t)pp.ni, (uint32_t)prm.a_chunks};
    return encode_f32_map(&prm.a_hi, hi, 4, dims, str, box) && encode_f32_map(&prm.a_lo, lo, 4, dims, str, box);
}
// Tensor maps of a chunk-major filter: dims [64, rows_pad/16, chunks], box = BN rows x 8 chunks.
static bool encode_filter_maps(TmaConvParams& prm, const float* hi, const float* lo, int rows_pad, int chunks, int bn,
                               int cls = 0) {
    const uint64_t dims[3] = {64, (uint64_t)rows_pad / 16, (uint64_t)chunks};
    const uint64_t str[2] = {256, (uint64_t)rows_pad * 16};
    const uint32_t box[3] = {64, (uint32_t)bn / 16, (uint32_t)TMA_KCH};
    return encode_f32_map(&prm.b_hi[cls], hi, 3, dims, str, box) && encode_f32_map(&prm.b_lo[cls], lo, 3, dims, str, box);
}
static void set_patch(TmaConvParams& prm, const PatchPlan& pp, int n_img, int Hv, int Wv) {
    prm.tw_log = pp.tw_log; prm.th_log = pp.th_log; prm.ni = pp.ni;
    prm.dPP.init((uint32_t)(pp.PH * pp.PW)); prm.dPW.init((uint32_t)pp.PW);
    prm.tm = (n_img + pp.ni - 1) / pp.ni * pp.PH * pp.PW;
    prm.n_img = n_img; prm.Hv = Hv; prm.Wv = Wv;
}
// Four consecutive rows of a tile are four consecutive, 16-byte aligned output floats.
static void set_vec_store(TmaConvParams& prm) {
    prm.vec_store = (prm.gxs == 1 && prm.ncls == 1 && prm.tw_log >= 2 && prm.Wv % 4 == 0 && prm.gys % 4 == 0 && prm.goff[0] % 4 == 0 &&
                     prm.img_stride % 4 == 0 && prm.nstr % 4 == 0 && (reinterpret_cast<uintptr_t>(prm.out) & 15) == 0)
                        ? 1 : 0;
}

// Forward convolution on the TMA engine.  *used = false (and FXB_OK) when the shapes cannot be
// described by tensor maps; the caller then takes the cp.async path.
// phase: which part of the call runs (FPROP_ALL, or one half for timing the two separately).
enum : int { FPROP_ALL = 0, FPROP_PREPASS_ONLY = 1, FPROP_MAIN_ONLY = 2 };
// Chaining of forward convolutions through class slabs: a layer can take its input slabs as written by the
// layer before it (no operand pass over X) and leave its own activated output as the slabs of the next layer.
struct FpropChain {
    const float* in_hi = nullptr;
    const float* in_lo = nullptr;
    SlabEmit emit;
    bool emitted = false;
};
// Bytes of the class-slab pair [hi | lo] of a layer's input; 0 when the layer does not read slabs.
static size_t conv_input_slab_bytes(const ConvGeom& g) {
    if (!tma_stride_ok(g) || g.CRS <= SMALLC_K || tensor_map_encoder() == nullptr) return 0;
    const TmaFpropLayout l = tma_fprop_layout(g);
    if (l.image_floats / 4 >= ((int64_t)1 << 31)) return 0;
    return 2 * align_up256((size_t)l.image_floats * 4);
}
static SlabEmit make_slab_emit(const ConvGeom& next, void* out) {
    const TmaFpropLayout l = tma_fprop_layout(next);
    SlabEmit e;
    e.hi = static_cast<float*>(out);
    e.lo = reinterpret_cast<float*>(static_cast<char*>(out) + align_up256((size_t)l.image_floats * 4));
    e.Q = l.Q; e.sw = next.sw; e.ph = next.ph; e.pw = next.pw; e.Wc = l.Wc;
    e.dsh.init((uint32_t)next.sh); e.dsw.init((uint32_t)next.sw);
    e.img_stride = (int64_t)l.Hc * l.Wc * 4;
    e.plane_stride = (int64_t)next.N * e.img_stride;
    return e;
}
static int launch_pack_xn(Context* c, const float* X, float* xn_hi, float* xn_lo, const ConvGeom& g, int Cp, int Hc, int Wc,
                          cudaStream_t st);
// xn_hi / xn_lo (optional): the operand pre-pass also leaves the filter-gradient kernel's packed input
// (xn_cp channels per cell) there, for a backward pass that follows.
static int conv_fprop_tma(Context* c, const float* X, const float* W, const float* bias, float* Y, const ConvGeom& g,
                          int act, void* ws, cudaStream_t st, bool* used, int phase = FPROP_ALL, float* xn_hi = nullptr,
                          float* xn_lo = nullptr, int xn_cp = 0, FpropChain* chain = nullptr) {
    *used = false;
    if (!tma_stride_ok(g) || tensor_map_encoder() == nullptr) return FXB_OK;
    const TmaFpropLayout l = tma_fprop_layout(g);
    if (l.image_floats / 4 >= ((int64_t)1 << 31)) return FXB_OK;
    const SplitWs w = carve_split_ws(ws, l.image_floats, l.filter_floats);
    const int bn = tile_cols(g.K);
    const PatchPlan pp = plan_patch(g.OH, g.OW);
    TmaConvParams prm;
    const bool slabs_given = chain != nullptr && chain->in_hi != nullptr;
    const float* a_hi = slabs_given ? chain->in_hi : w.a_hi;
    const float* a_lo = slabs_given ? chain->in_lo : w.a_lo;
    if (!encode_slab_maps(prm, a_hi, a_lo, l.Wc, l.Hc, l.planes, g.N, pp, l.Q)) return FXB_OK;
    if (!encode_filter_maps(prm, w.b_hi, w.b_lo, l.rows_pad, g.RS * l.Q, bn)) return FXB_OK;
    *used = true;
    if (phase != FPROP_MAIN_ONLY) {
        int rc = FXB_OK;
        if (!slabs_given) {  // (otherwise the layer before this one has written them from its epilogue)
            const int64_t total = l.image_floats / 4 / g.sw;  // one thread per cell of all x classes
            const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)c->sm_count * 16);
            split_image_to_class_slabs_kernel<<<blocks, 256, 0, st>>>(X, w.a_hi, w.a_lo, g.C, g.H, g.W, l.Q, g.sh, g.sw, g.ph,
                                                                      g.pw, total, FastDiv((uint32_t)l.Wc), FastDiv((uint32_t)l.Hc),
                                                                      FastDiv((uint32_t)g.N), FastDiv((uint32_t)l.Q), g.N, l.Hc, l.Wc);
            rc = launch_status(c, "split_image_to_class_slabs_kernel");
            if (rc) return rc;
        }
        if (xn_hi != nullptr) {  // (a single pass writing both layouts measured slower than the two passes)
            rc = launch_pack_xn(c, X, xn_hi, xn_lo, g, xn_cp, l.Hc, l.Wc, st);
            if (rc) return rc;
        }
        FilterClassBase fc{};
        const int ftotal = g.RS * l.Q * l.rows_pad;
        const int fblocks = std::max(1, std::min((ftotal + 255) / 256, c->sm_count * 8));
        split_filter_chunk_major_kernel<<<fblocks, 256, 0, st>>>(W, w.b_hi, w.b_lo, g.K, g.C, g.R, g.S, l.Q, g.K, l.rows_pad, 0, 1, 1, fc);
        rc = launch_status(c, "split_filter_chunk_major_kernel");
        if (rc) return rc;
    }
    if (phase == FPROP_PREPASS_ONLY) return FXB_OK;
    set_patch(prm, pp, g.N, g.OH, g.OW);
    prm.tn = (g.K + bn - 1) / bn;
    prm.ncols = g.K;
    prm.ncls = 1;
    prm.kchunks[0] = g.RS * l.Q;
    prm.three_pass = c->math_mode == FXB_MATH_3XTF32 ? 1 : 0;
    prm.drain_group = c->drain_group;
    prm.dQ.init((uint32_t)l.Q); prm.dS[0].init((uint32_t)g.S);
    prm.Q = l.Q; prm.sh = g.sh; prm.sw = g.sw; prm.dir = 1; prm.by[0] = 0; prm.bx[0] = 0; prm.planes = l.planes;
    prm.out = Y; prm.bias = bias; prm.act = act;
    prm.img_stride = (int64_t)g.K * g.P; prm.nstr = g.P; prm.goff[0] = 0; prm.gys = g.OW; prm.gxs = 1;
    const FpropSplit fs = fprop_split_plan(c, g);
    if (fs.splits > 1) {
        prm.splits = fs.splits;
        prm.stages_per_split = fs.stages_per_split;
        prm.split_stride = (int64_t)g.N * g.K * g.P;
        prm.out = reinterpret_cast<float*>(static_cast<char*>(ws) + align_up256(w.bytes));
    }
    set_vec_store(prm);
    // several column tiles: walk them row-tile group by row-tile group, so that the second column tile finds the
    // image tiles of the first one still in L2
    if (prm.tn > 1 && fs.splits == 1) prm.group_m = 8;
    if (chain != nullptr && chain->emit.hi != nullptr && fs.splits == 1) {
        prm.emit = chain->emit;
        chain->emitted = true;
    }
    int rc = launch_tma(c, prm, bn, st);
    if (rc || fs.splits == 1) return rc;
    const int64_t n = prm.split_stride;
    const int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)c->sm_count * 8);
    splitk_bias_act_kernel<<<blocks, 256, 0, st>>>(prm.out, Y, n, n, fs.splits, bias, FastDiv((uint32_t)g.P), g.K, act);
    return launch_status(c, "splitk_bias_act_kernel");
}

// ---- GEMM on the same engine: C[M,N] = act(op(A) . op(B) + bias) is the forward pass of a 1x1 convolution
// over M images of one pixel: the row operand is the slab tensor S[K/4][M][4], the column operand a
// chunk-major "filter" F[K/4][N][4]; both come from one split pass per operand, which also absorbs
// the transposes.  Tiles are walked in groups of 16 row tiles so that the CTAs running side by side
// share operand rows in L2.
static bool tma_gemm_wanted(const Context* c, int64_t M, int64_t N, int64_t K) {
    if (M < 128 || N < 64 || K < 128 || tensor_map_encoder() == nullptr) return false;
    const int64_t K4 = (K + 3) / 4;
    if (!fits_i32(K4 * 4) || !fits_i32(M + 128) || !fits_i32(N + 128)) return false;
    const int bn = tile_cols((int)std::min<int64_t>(N, 128));
    const int64_t tiles = ((M + 127) / 128) * ((N + bn - 1) / bn);
    return tiles >= c->sm_count / 2 && tiles < ((int64_t)1 << 30);
}
static size_t tma_gemm_bytes(int64_t M, int64_t N, int64_t K) {
    const int64_t K4 = (K + 3) / 4;
    const int bn = tile_cols((int)std::min<int64_t>(N, 128));
    const int64_t rows_pad = (N + bn - 1) / bn * bn;
    return carve_split_ws(nullptr, K4 * ((M + 15) / 16 * 16) * 4, K4 * rows_pad * 4).bytes;
}
static int launch_split_matrix(Context* c, const float* x, const float* aux, int64_t ld, bool rows_contiguous, int rows, int K,
                               int rows_pad, float* hi, float* lo, int act, cudaStream_t st) {
    const int K4 = (K + 3) / 4;
    if (rows_contiguous) {
        const int64_t total = (int64_t)K4 * rows_pad;
        const int blocks = (int)std::min<int64_t>((total + 255) / 256, (int64_t)c->sm_count * 16);
        split_matrix_rowmajor_kernel<<<blocks, 256, 0, st>>>(x, aux, ld, rows, K, rows_pad, total, hi, lo, aux ? act : FXB_ACT_NONE,
                                                             c->sigmoid_grad_math);
        return launch_status(c, "split_matrix_rowmajor_kernel");
    }
    const bool vec_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (aux == nullptr || (reinterpret_cast<uintptr_t>(aux) & 15) == 0) &&
                        ld % 4 == 0;
    const int gy = (K4 + 31) / 32;
    if (gy > 65535) return fail(c, FXB_ERR_UNSUPPORTED, "Matrix multiplication: K above 8 million is not supported on this path");
    dim3 grid((unsigned)((rows_pad + 31) / 32), (unsigned)gy);
    split_matrix_kmajor_kernel<<<grid, 256, 0, st>>>(x, aux, ld, rows, K, K4, rows_pad, hi, lo, vec_ok ? 1 : 0,
                                                     aux ? act : FXB_ACT_NONE, c->sigmoid_grad_math);
    return launch_status(c, "split_matrix_kmajor_kernel");
}
static int gemm_tma(Context* c, int ta, int tb, int64_t M, int64_t N, int64_t K, const float* A, int64_t lda, const float* B,
                    int64_t ldb, float* C, int64_t ldc, const float* bias, int act, const float* a_aux, int a_act, void* ws,
                    cudaStream_t st, bool* used) {
    *used = false;
    const int K4 = (int)((K + 3) / 4);
    const int bn = tile_cols((int)std::min<int64_t>(N, 128));
    const int rows_pad = round_up((int)N, bn);
    const int Mp = round_up((int)M, 16);
    const SplitWs w = carve_split_ws(ws, (int64_t)K4 * Mp * 4, (int64_t)K4 * rows_pad * 4);
    TmaConvParams prm;
    {
        // row operand: 16 rows x 4 floats form the innermost 256 bytes (long copy lines): dims [64, 1, Mp/16, K/4];
        // one box = 8 row groups x 8 chunks = the 128 x 32 stage
        const uint64_t dims[4] = {64, 1, (uint64_t)Mp / 16, (uint64_t)K4};
        const uint64_t str[3] = {256, 256, (uint64_t)Mp * 16};
        const uint32_t box[4] = {64, 1, 8, (uint32_t)TMA_KCH};
        if (!encode_f32_map(&prm.a_hi, w.a_hi, 4, dims, str, box) || !encode_f32_map(&prm.a_lo, w.a_lo, 4, dims, str, box))
            return FXB_OK;
        prm.a_chunks = TMA_KCH;
        prm.a_nshift = 4;
    }
    if (!encode_filter_maps(prm, w.b_hi, w.b_lo, rows_pad, K4, bn)) return FXB_OK;
    *used = true;
    // op(A)(m, k): trans_a == 0 -> A[m * lda + k] (K contiguous); trans_a == 1 -> A[k * lda + m].
    int rc = launch_split_matrix(c, A, a_aux, lda, ta != 0, (int)M, (int)K, Mp, w.a_hi, w.a_lo, a_act, st);
    if (rc) return rc;
    // op(B)(k, n): trans_b == 0 -> B[k * ldb + n] (columns contiguous); trans_b == 1 -> B[n * ldb + k].
    rc = launch_split_matrix(c, B, nullptr, ldb, tb == 0, (int)N, (int)K, rows_pad, w.b_hi, w.b_lo, FXB_ACT_NONE, st);
    if (rc) return rc;
    PatchPlan pp;
    pp.tw_log = 0; pp.th_log = 0; pp.ni = 128; pp.PW = 1; pp.PH = 1;
    set_patch(prm, pp, (int)M, 1, 1);
    prm.tn = ((int)N + bn - 1) / bn;
    prm.ncols = (int)N;
    prm.ncls = 1;
    prm.kchunks[0] = K4;
    prm.three_pass = c->math_mode == FXB_MATH_3XTF32 ? 1 : 0;
    prm.drain_group = c->drain_group;
    prm.dQ.init((uint32_t)K4); prm.dS[0].init(1);
    prm.Q = K4; prm.sh = 1; prm.sw = 1; prm.dir = 1; prm.by[0] = 0; prm.bx[0] = 0; prm.planes = K4;
    prm.out = C; prm.bias = bias; prm.act = act;
    prm.img_stride = ldc; prm.nstr = 1; prm.goff[0] = 0; prm.gys = 0; prm.gxs = 0;
    prm.vec_store = 0;
    prm.row_vec = (ldc % 4 == 0 && N % 4 == 0 && (reinterpret_cast<uintptr_t>(C) & 15) == 0) ? 1 : 0;
    prm.group_m = 16;
    return launch_tma(c, prm, bn, st);
}

static int conv_fprop_async(Context* c, const float* X, const float* W, const float* bias, float* Y, const ConvGeom& g,
                            int act, void* ws, cudaStream_t st) {
    const int C4 = (g.C + 3) / 4;
    const SplitWs w = carve_split_ws(ws, (int64_t)g.N * C4 * g.HW * 4, (int64_t)g.K * g.RS * C4 * 4);
    int rc = launch_split_image(c, X, nullptr, w.a_hi, w.a_lo, g.N, g.C, g.HW, FXB_ACT_NONE, st);
    if (rc) return rc;
    rc = launch_split_filter(c, W, w.b_hi, w.b_lo, g.K, g.C, g.RS, false, st);
    if (rc) return rc;
    SlabPixelLoader la;
    la.hi = w.a_hi; la.lo = w.a_lo; la.C4 = C4; la.Hs = g.H; la.Ws = g.W; la.plane4 = g.HW * 4;
    la.nR = g.R; la.nS = g.S; la.dir = 1; la.rows = g.N * g.P; la.kchunks = g.RS * C4;
    la.dHaWa.init((uint32_t)g.P); la.dWa.init((uint32_t)g.OW); la.dC4.init((uint32_t)C4); la.dS.init((uint32_t)g.S);
    la.ay = g.sh; la.by = -g.ph; la.ax = g.sw; la.bx = -g.pw;
    SplitDenseLoader lb;
    lb.hi = w.b_hi; lb.lo = w.b_lo; lb.ld = (int64_t)g.RS * C4 * 4; lb.rows = g.K; lb.kchunks = g.RS * C4;
    lb.remap = 0; lb.Q = 1; lb.S_full = 1; lb.cy = lb.cx = 0; lb.sh = lb.sw = 1; lb.dQ.init(1); lb.dSc.init(1);
    Problem<float> p;
    p.M = g.N * g.P; p.N = g.K; p.K = g.RS * C4 * 4;
    auto ow = make_plane_writer<float>(Y, g.P, (int64_t)g.K * g.P, bias, act, p.M, p.N);
    return launch_contract(c, la, lb, ow, p, st);
}

template <typename T>
static int conv_fprop_impl(Context* c, const T* X, const T* W, const T* bias, T* Y, const fxb_conv2d_desc* d, int act,
                           void* ws, size_t ws_bytes, cudaStream_t st, int phase = FPROP_ALL, FpropChain* chain = nullptr) {
    ConvGeom g;
    int rc = make_geom(c, d, g);
    if (rc) return rc;
    FXB_CHECK_ARG(c, X && W && Y, "Conv2D got a null buffer");
    FXB_CHECK_ARG(c, act >= FXB_ACT_NONE && act <= FXB_ACT_TANH, "Unknown activation code");
    if (phase != FPROP_ALL) {
        // one half only: nothing but the tensor-map path has two halves
        if constexpr (sizeof(T) == 4) {
            bool used = false;
            if (c->operand_path == FXB_PATH_AUTO && ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255) == 0 &&
                ws_bytes >= fprop_split_bytes(c, g) && g.CRS > SMALLC_K)
                rc = conv_fprop_tma(c, X, W, bias, Y, g, act, ws, st, &used, phase);
            if (rc) return rc;
            if (used) return FXB_OK;
        }
        return fail(c, FXB_ERR_UNSUPPORTED, "this convolution has no separate operand pre-pass");
    }
    if (c->operand_path == FXB_PATH_AUTO && g.CRS <= SMALLC_K && (size_t)g.K * SMALLC_K * sizeof(T) <= 48 * 1024) {
        // a handful of input values per output: one thread per output pixel on the CUDA cores (the tensor-map
        // path measured slower here: conv 3->64 on 1024 x 32 x 32 takes 0.225 ms there against 0.188 ms, its
        // two-stage tiles are bound by the drain + epilogue of 8192 tiles)
        const int64_t npix = (int64_t)g.N * g.P;
        const unsigned blocks = (unsigned)((npix + 255) / 256);
        const size_t smem = (size_t)g.K * SMALLC_K * sizeof(T);
        if constexpr (sizeof(T) == 4) {
            if (chain != nullptr && chain->emit.hi != nullptr) {
                chain->emitted = true;
                smallc_conv_fwd_kernel<T, true><<<blocks, 256, smem, st>>>(X, W, bias, Y, g, npix, act, chain->emit);
                return launch_status(c, "smallc_conv_fwd_kernel");
            }
        }
        smallc_conv_fwd_kernel<T, false><<<blocks, 256, smem, st>>>(X, W, bias, Y, g, npix, act, SlabEmit{});
        return launch_status(c, "smallc_conv_fwd_kernel");
    }
    if constexpr (sizeof(T) == 4) {
        // With a workspace the operands are pre-split once and copied by the tensor-map engine (or, for
        // shapes it cannot describe, by cp.async); without one the kernel gathers and splits them on
        // the fly (same results).
        if (c->operand_path != FXB_PATH_GATHER && ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255) == 0 &&
            ws_bytes >= fprop_split_bytes(c, g)) {
            if (c->operand_path != FXB_PATH_CP_ASYNC) {
                bool used = false;
                rc = conv_fprop_tma(c, X, W, bias, Y, g, act, ws, st, &used, FPROP_ALL, nullptr, nullptr, 0, chain);
                if (rc || used) return rc;
            }
            return conv_fprop_async(c, X, W, bias, Y, g, act, ws, st);
        }
    }
    Im2colLoader<T> la;
    la.x = X; la.g = g; la.rows = g.N * g.P;
    auto lb = make_dense<T, true>(c, W, g.CRS, g.K, g.CRS, nullptr, 0);
    Problem<T> p;
    p.M = g.N * g.P; p.N = g.K; p.K = g.CRS;
    auto ow = make_plane_writer<T>(Y, g.P, (int64_t)g.K * g.P, bias, act, p.M, p.N);
    return launch_contract(c, la, lb, ow, p, st);
}

// One stride-residue class of input pixels (the set that shares the same filter taps).
static bool dgrad_class(const ConvGeom& g, int cy, int cx, DgradClass& cl) {
    cl.cy = cy; cl.cx = cx;
    cl.y0 = ((cy - g.ph) % g.sh + g.sh) % g.sh;
    cl.x0 = ((cx - g.pw) % g.sw + g.sw) % g.sw;
    cl.Hc = cl.y0 < g.H ? (g.H - cl.y0 + g.sh - 1) / g.sh : 0;
    cl.Wc = cl.x0 < g.W ? (g.W - cl.x0 + g.sw - 1) / g.sw : 0;
    if (cl.Hc == 0 || cl.Wc == 0) return false;
    cl.Rc = cy < g.R ? (g.R - cy + g.sh - 1) / g.sh : 0;
    cl.Sc = cx < g.S ? (g.S - cx + g.sw - 1) / g.sw : 0;
    cl.oy0 = (cl.y0 + g.ph - cy) / g.sh;
    cl.ox0 = (cl.x0 + g.pw - cx) / g.sw;
    cl.finish();
    return true;
}

// Input gradient on the TMA engine: dZ = dY * act'(Y) as hi / lo channel slabs, the filter chunk-major
// and grouped by stride-residue class, one launch per class.  *used = false when some class cannot be
// described by tensor maps (nothing has been launched then).
static int conv_dgrad_tma(Context* c, const float* dY, const float* Yact, const float* W, float* dX, const ConvGeom& g,
                          int act, void* ws, cudaStream_t st, bool* used, bool slabs_ready = false) {
    *used = false;
    if (!tma_stride_ok(g) || tensor_map_encoder() == nullptr) return FXB_OK;
    const int K4 = (g.K + 3) / 4;
    const int bn = tile_cols(g.C);
    const int rows_pad = round_up(g.C, bn);
    const SplitWs w = carve_split_ws(ws, (int64_t)g.N * K4 * g.P * 4, (int64_t)rows_pad * g.RS * K4 * 4);
    FilterClassBase fc{};
    TmaConvParams prm[16];
    bool live[16] = {};
    int chunk_base = 0;
    for (int cy = 0; cy < g.sh; ++cy)
        for (int cx = 0; cx < g.sw; ++cx) {
            const int ci = cy * g.sw + cx;
            DgradClass cl;
            const bool has_pixels = dgrad_class(g, cy, cx, cl);
            const int Rc = cy < g.R ? (g.R - cy + g.sh - 1) / g.sh : 0, Sc = cx < g.S ? (g.S - cx + g.sw - 1) / g.sw : 0;
            const int chunks = Rc * Sc * K4;
            fc.base[ci] = chunk_base;
            chunk_base += chunks;
            if (!has_pixels) continue;
            if (chunks == 0) return FXB_OK;  // a class without taps (all zeros): left to the general path
            const PatchPlan pp = plan_patch(cl.Hc, cl.Wc);
            TmaConvParams& q = prm[ci];
            if (!encode_slab_maps(q, w.a_hi, w.a_lo, g.OW, g.OH, K4, g.N, pp, K4)) return FXB_OK;
            const int64_t boff = (int64_t)fc.base[ci] * rows_pad * 4;
            if (!encode_filter_maps(q, w.b_hi + boff, w.b_lo + boff, rows_pad, chunks, bn)) return FXB_OK;
            set_patch(q, pp, g.N, cl.Hc, cl.Wc);
            q.tn = (g.C + bn - 1) / bn;
            q.ncols = g.C;
            q.ncls = 1;
            if (q.tn > 1) q.group_m = 8;  // (as in the forward pass: column tiles of a row-tile group back to back)
            q.kchunks[0] = chunks;
            q.three_pass = c->math_mode == FXB_MATH_3XTF32 ? 1 : 0;
            q.drain_group = c->drain_group;
            q.dQ.init((uint32_t)K4); q.dS[0].init((uint32_t)Sc);
            q.Q = K4; q.sh = 1; q.sw = 1; q.dir = -1; q.by[0] = cl.oy0; q.bx[0] = cl.ox0; q.planes = K4;
            q.out = dX; q.bias = nullptr; q.act = FXB_ACT_NONE;
            q.img_stride = (int64_t)g.C * g.HW; q.nstr = g.HW;
            q.goff[0] = (int64_t)cl.y0 * g.W + cl.x0; q.gys = (int64_t)g.sh * g.W; q.gxs = g.sw;
            set_vec_store(q);
            live[ci] = true;
        }
    *used = true;
    int rc = FXB_OK;
    if (!slabs_ready) {  // (the fused backward's operand pass has written the dZ slabs already)
        rc = launch_split_image(c, dY, act == FXB_ACT_NONE ? nullptr : Yact, w.a_hi, w.a_lo, g.N, g.K, g.P, act, st, true);
        if (rc) return rc;
    }
    const int ftotal = g.RS * K4 * rows_pad;
    const int fblocks = std::max(1, std::min((ftotal + 255) / 256, c->sm_count * 8));
    split_filter_chunk_major_kernel<<<fblocks, 256, 0, st>>>(W, w.b_hi, w.b_lo, g.K, g.C, g.R, g.S, K4, g.C, rows_pad, 1, g.sh, g.sw, fc);
    rc = launch_status(c, "split_filter_chunk_major_kernel");
    if (rc) return rc;
    // Classes with the same grid are merged into one launch, class index fastest in the item order: the CTAs
    // that run side by side then write the interleaved pixels of the same patch, and the partial sectors of
    // the strided stores meet in L2 instead of travelling to DRAM once per class.
    int order[16], nl = 0;
    bool uniform = true;
    for (int ci = 0; ci < g.sh * g.sw; ++ci) {
        if (!live[ci]) continue;
        if (nl > 0 && (prm[ci].Hv != prm[order[0]].Hv || prm[ci].Wv != prm[order[0]].Wv || prm[ci].tm != prm[order[0]].tm))
            uniform = false;
        order[nl++] = ci;
    }
    if (uniform && nl >= 2 && nl <= TMA_MAX_CLS) {
        TmaConvParams m = prm[order[0]];
        for (int j = 1; j < nl; ++j) {
            const TmaConvParams& q = prm[order[j]];
            m.b_hi[j] = q.b_hi[0]; m.b_lo[j] = q.b_lo[0];
            m.kchunks[j] = q.kchunks[0]; m.dS[j] = q.dS[0];
            m.by[j] = q.by[0]; m.bx[j] = q.bx[0]; m.goff[j] = q.goff[0];
        }
        m.ncls = nl;
        m.vec_store = 0;
        return launch_tma(c, m, bn, st);
    }
    for (int j = 0; j < nl; ++j) {
        rc = launch_tma(c, prm[order[j]], bn, st);
        if (rc) return rc;
    }
    return FXB_OK;
}

template <typename T>
static int conv_dgrad_impl(Context* c, const T* dY, const T* Yact, const T* W, T* dX, const fxb_conv2d_desc* d, int act,
                           void* ws, size_t ws_bytes, cudaStream_t st) {
    ConvGeom g;
    int rc = make_geom(c, d, g);
    if (rc) return rc;
    FXB_CHECK_ARG(c, dY && W && dX, "Conv2d backward got a null buffer");
    FXB_CHECK_ARG(c, act == FXB_ACT_NONE || Yact != nullptr, "Fused activation backward needs the layer output");
    bool use_async = false;
    SplitWs sw{};
    const int K4 = (g.K + 3) / 4;
    if constexpr (sizeof(T) == 4) {
        if (c->operand_path == FXB_PATH_AUTO && ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255) == 0 &&
            ws_bytes >= dgrad_split_bytes(g)) {
            bool used = false;
            rc = conv_dgrad_tma(c, reinterpret_cast<const float*>(dY), reinterpret_cast<const float*>(Yact),
                                reinterpret_cast<const float*>(W), reinterpret_cast<float*>(dX), g, act, ws, st, &used);
            if (rc || used) return rc;
        }
        if (c->operand_path != FXB_PATH_GATHER && ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255) == 0 &&
            ws_bytes >= dgrad_split_bytes(g)) {
            // dZ = dY * act'(Y) is formed once here instead of once per filter tap in the main kernel.
            sw = carve_split_ws(ws, (int64_t)g.N * K4 * g.P * 4, (int64_t)g.C * g.RS * K4 * 4);
            rc = launch_split_image(c, reinterpret_cast<const float*>(dY), act == FXB_ACT_NONE ? nullptr : reinterpret_cast<const float*>(Yact),
                                    sw.a_hi, sw.a_lo, g.N, g.K, g.P, act, st);
            if (rc) return rc;
            rc = launch_split_filter(c, reinterpret_cast<const float*>(W), sw.b_hi, sw.b_lo, g.K, g.C, g.RS, true, st);
            if (rc) return rc;
            use_async = true;
        }
    }
    // One launch per stride-residue class of input pixels (a single class when stride is 1).
    for (int cy = 0; cy < g.sh; ++cy) {
        for (int cx = 0; cx < g.sw; ++cx) {
            DgradClass cl;
            cl.cy = cy; cl.cx = cx;
            cl.y0 = ((cy - g.ph) % g.sh + g.sh) % g.sh;
            cl.x0 = ((cx - g.pw) % g.sw + g.sw) % g.sw;
            cl.Hc = cl.y0 < g.H ? (g.H - cl.y0 + g.sh - 1) / g.sh : 0;
            cl.Wc = cl.x0 < g.W ? (g.W - cl.x0 + g.sw - 1) / g.sw : 0;
            if (cl.Hc == 0 || cl.Wc == 0) continue;
            cl.Rc = cy < g.R ? (g.R - cy + g.sh - 1) / g.sh : 0;
            cl.Sc = cx < g.S ? (g.S - cx + g.sw - 1) / g.sw : 0;
            cl.oy0 = (cl.y0 + g.ph - cy) / g.sh;
            cl.ox0 = (cl.x0 + g.pw - cx) / g.sw;
            cl.finish();
            if constexpr (sizeof(T) == 4) {
                if (use_async) {
                    SlabPixelLoader la;
                    la.hi = sw.a_hi; la.lo = sw.a_lo; la.C4 = K4; la.Hs = g.OH; la.Ws = g.OW; la.plane4 = g.P * 4;
                    la.nR = cl.Rc; la.nS = cl.Sc; la.dir = -1; la.rows = g.N * cl.Hc * cl.Wc; la.kchunks = cl.Rc * cl.Sc * K4;
                    la.dHaWa.init((uint32_t)(cl.Hc * cl.Wc)); la.dWa.init((uint32_t)cl.Wc); la.dC4.init((uint32_t)K4);
                    la.dS.init((uint32_t)(cl.Sc > 0 ? cl.Sc : 1));
                    la.ay = 1; la.by = cl.oy0; la.ax = 1; la.bx = cl.ox0;
                    SplitDenseLoader lb;
                    lb.hi = sw.b_hi; lb.lo = sw.b_lo; lb.ld = (int64_t)g.RS * K4 * 4; lb.rows = g.C; lb.kchunks = la.kchunks;
                    lb.remap = 1; lb.Q = K4; lb.S_full = g.S; lb.cy = cy; lb.cx = cx; lb.sh = g.sh; lb.sw = g.sw;
                    lb.dQ.init((uint32_t)K4); lb.dSc.init((uint32_t)(cl.Sc > 0 ? cl.Sc : 1));
                    Problem<float> p;
                    p.M = la.rows; p.N = g.C; p.K = la.kchunks * 4;
                    auto ow = make_plane_writer<float>(reinterpret_cast<float*>(dX), cl.Hc * cl.Wc, (int64_t)g.C * g.HW, nullptr,
                                                       FXB_ACT_NONE, p.M, p.N);
                    ow.nstr = g.HW;
                    ow.gw = cl.Wc; ow.dgw.init((uint32_t)cl.Wc);
                    ow.goff = (int64_t)cl.y0 * g.W + cl.x0; ow.gys = (int64_t)g.sh * g.W; ow.gxs = g.sw;
                    rc = launch_contract(c, la, lb, ow, p, st);
                    if (rc) return rc;
                    continue;
                }
            }
            DgradLoader<T> la;
            la.dy = dY; la.aux = act == FXB_ACT_NONE ? nullptr : Yact; la.g = g; la.cl = cl;
            la.rows = g.N * cl.Hc * cl.Wc; la.Ktot = g.K * cl.Rc * cl.Sc;
            la.act = act; la.sig_math = c->sigmoid_grad_math;
            DgradFilterLoader<T> lb;
            lb.w = W; lb.g = g; lb.cl = cl; lb.Ktot = la.Ktot;
            Problem<T> p;
            p.M = la.rows; p.N = g.C; p.K = la.Ktot;
            auto ow = make_plane_writer<T>(dX, cl.Hc * cl.Wc, (int64_t)g.C * g.HW, nullptr, FXB_ACT_NONE, p.M, p.N);
            ow.nstr = g.HW;
            ow.gw = cl.Wc; ow.dgw.init((uint32_t)cl.Wc);
            ow.goff = (int64_t)cl.y0 * g.W + cl.x0; ow.gys = (int64_t)g.sh * g.W; ow.gxs = g.sw;
            rc = launch_contract(c, la, lb, ow, p, st);
            if (rc) return rc;
        }
    }
    return FXB_OK;
}

// ---- small-C filter gradient: partial sums of every block, then a fixed-order finish ---------
static int smallc_wgrad_blocks(const Context* c, int64_t npix) {
    // at least eight 32-pixel tiles per block (the finish kernels add one row per block), at most eight blocks per SM
    return (int)std::max<int64_t>(1, std::min<int64_t>((npix + 255) / 256, (int64_t)c->sm_count * 8));
}
static size_t smallc_wgrad_bytes(const Context* c, int64_t npix, size_t elem) {
    const size_t blocks = (size_t)smallc_wgrad_blocks(c, npix);
    return blocks * (64 * SMALLC_K + 64) * elem;
}
// db[o] = sum over blocks of dbpart[b][o] (rows of 64), same fixed tree as the filter finish.
template <typename T>
__global__ void __launch_bounds__(256) smallc_db_finish_kernel(const T* __restrict__ dbpart, T* __restrict__ db, int K, int rows) {
    __shared__ T red[8][32];
    const int el = threadIdx.x & 31, bl = threadIdx.x >> 5;
    const int o = blockIdx.x * 32 + el;
    T a0 = T(0), a1 = T(0), a2 = T(0), a3 = T(0);
    int b = bl;
    for (; b + 24 < rows; b += 32) {  // four independent loads in flight
        a0 += __ldg(dbpart + (int64_t)b * 64 + o);
        a1 += __ldg(dbpart + (int64_t)(b + 8) * 64 + o);
        a2 += __ldg(dbpart + (int64_t)(b + 16) * 64 + o);
        a3 += __ldg(dbpart + (int64_t)(b + 24) * 64 + o);
    }
    for (; b < rows; b += 8) a0 += __ldg(dbpart + (int64_t)b * 64 + o);
    red[bl][el] = (a0 + a1) + (a2 + a3);
    __syncthreads();
    if (bl == 0 && o < K)
        db[o] = ((red[0][el] + red[1][el]) + (red[2][el] + red[3][el])) + ((red[4][el] + red[5][el]) + (red[6][el] + red[7][el]));
}

// ---- tensor-map filter-gradient path ---------------------------------------------------------
// Geometry and workspace plan.  Workspace order: [DZN hi | DZN lo | XN hi | XN lo | split-K partials | db partials];
// the XN pair is left out when the caller brings its own (prepared by the forward pass).
struct TmaWgradLayout {
    bool ok;
    int Kp, Cp, Cb, tpt, cblocks, n4, ncls, Hc, Wc, bw, bh, PWs, PHs, spg, tm, tn, splits, stages_total, stages_per_split;
    int pblocks, db_rows;
    int64_t dz_floats, xn_floats, part_floats, dbpart_floats;
    size_t bytes, bytes_without_xn;
};
static TmaWgradLayout tma_wgrad_layout(const Context* c, const ConvGeom& g) {
    TmaWgradLayout l{};
    l.ok = false;
    if (!tma_stride_ok(g) || g.S > 32 || g.R > 32) return l;
    l.Cp = round_up(g.C, 16);
    if (l.Cp > 128) l.Cp = round_up(g.C, 128);
    else if (l.Cp > 64) l.Cp = 128;
    else if (l.Cp > 32) l.Cp = 64;
    else if (l.Cp > 16) l.Cp = 32;
    l.Cb = std::min(l.Cp, 128);
    // Few input channels mean many narrow (N = 16 or 32) MMAs per stage, each re-reading the whole dZ
    // tile from shared memory: measured slower than the gather path, which therefore keeps those layers.
    if (l.Cb < 64) return l;
    l.tpt = 128 / l.Cb;
    l.cblocks = std::max(1, l.Cp / 128);
    l.Kp = round_up(g.K, 16);
    l.n4 = (g.N + 3) / 4;
    l.ncls = g.sh * g.sw;
    l.Hc = (g.H - 1 + g.ph) / g.sh + 1;
    l.Wc = (g.W - 1 + g.pw) / g.sw + 1;
    l.bw = std::min(TMA_KCH, 1 << log2_ceil(g.OW));
    l.bh = TMA_KCH / l.bw;
    l.PWs = (g.OW + l.bw - 1) / l.bw;
    l.PHs = (g.OH + l.bh - 1) / l.bh;
    l.spg = l.PWs * l.PHs;
    const int64_t stages = (int64_t)l.n4 * l.spg;
    if (stages >= ((int64_t)1 << 30) || (int64_t)l.ncls * l.n4 >= ((int64_t)1 << 30)) return l;
    l.stages_total = (int)stages;
    l.tm = (g.K + 127) / 128;
    l.tn = l.cblocks > 1 ? g.RS * l.cblocks : (g.RS + l.tpt - 1) / l.tpt;
    const int tiles = l.tm * l.tn;
    int splits = std::max(1, std::min(l.stages_total / 8, c->sm_count / tiles));  // one wave of CTAs
    l.stages_per_split = (l.stages_total + splits - 1) / splits;
    l.splits = (l.stages_total + l.stages_per_split - 1) / l.stages_per_split;
    l.pblocks = (g.P + 31) / 32;
    l.db_rows = l.n4 * l.pblocks;
    l.dz_floats = (int64_t)l.n4 * g.P * l.Kp * 4;
    l.xn_floats = (int64_t)l.ncls * l.n4 * l.Hc * l.Wc * l.Cp * 4;
    if (l.dz_floats >= ((int64_t)1 << 33) || l.xn_floats >= ((int64_t)1 << 33)) return l;
    l.part_floats = l.splits > 1 ? (int64_t)l.splits * g.K * g.CRS : 0;
    l.dbpart_floats = (int64_t)l.db_rows * g.K;
    l.bytes_without_xn = 2 * align_up256((size_t)l.dz_floats * 4) + align_up256((size_t)l.part_floats * 4) +
                         align_up256((size_t)l.dbpart_floats * 4);
    l.bytes = l.bytes_without_xn + 2 * align_up256((size_t)l.xn_floats * 4);
    l.ok = true;
    return l;
}

// x -> XN, the packed input of the filter-gradient kernel.
static int launch_pack_xn(Context* c, const float* X, float* xn_hi, float* xn_lo, const ConvGeom& g, int Cp, int Hc, int Wc,
                          cudaStream_t st) {
    const int n4 = (g.N + 3) / 4;
    const int Wp = Wc * g.sw, Hp = Hc * g.sh;
    // Rows per block: the band height that minimises (waves of blocks at four blocks per SM) x (32-cell chunks per
    // block + a fixed cost), so that the last wave is not mostly empty (at most about eight chunks per block).
    const int gx = (Cp + XN_CT - 1) / XN_CT;
    int ry = 1;
    double best = 1e300;
    for (int r = 1; r <= Hp && (r == 1 || r * Wp <= 288); ++r) {
        const int64_t blocks = (int64_t)gx * ((Hp + r - 1) / r) * n4;
        const int64_t waves = (blocks + (int64_t)c->sm_count * 4 - 1) / ((int64_t)c->sm_count * 4);
        const double cost = (double)waves * ((r * Wp + 31) / 32 + 0.5);
        if (cost < best) { best = cost; ry = r; }
    }
    if (n4 > 65535 || (Hp + ry - 1) / ry > 65535) return fail(c, FXB_ERR_UNSUPPORTED, "Conv2D batch too large for the packed operand pass");
    dim3 grid(gx, (Hp + ry - 1) / ry, n4);
    static bool carveout_set[64] = {};
    if (!carveout_set[c->device & 63]) {  // 34 KB of static shared memory per block: ask for room for four blocks per SM
        FXB_CUDA_OK(c, cudaFuncSetAttribute(pack_xn_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        carveout_set[c->device & 63] = true;
    }
    pack_xn_kernel<<<grid, 256, 0, st>>>(X, xn_hi, xn_lo, g.N, g.C, Cp, g.H, g.W, g.ph, g.pw, Hc, Wc, n4, ry, FastDiv((uint32_t)Wp),
                                         FastDiv((uint32_t)g.sh), FastDiv((uint32_t)g.sw));
    return launch_status(c, "pack_xn_kernel");
}
// dY (* act'(Y)) -> DZN (+ channel slabs for the input gradient) (+ bias gradient).
static int launch_pack_dz(Context* c, const float* dY, const float* Yact, float* dzn_hi, float* dzn_lo, float* slab_hi,
                          float* slab_lo, float* dbpart, float* db, const ConvGeom& g, const TmaWgradLayout& l, int act,
                          cudaStream_t st) {
    if (l.n4 > 65535 || (l.Kp + 31) / 32 > 65535) return fail(c, FXB_ERR_UNSUPPORTED, "Conv2D batch too large for the packed operand pass");
    dim3 grid(l.pblocks, (l.Kp + 31) / 32, l.n4);
    pack_dz_kernel<<<grid, 256, 0, st>>>(dY, act == FXB_ACT_NONE ? nullptr : Yact, dzn_hi, dzn_lo, slab_hi, slab_lo,
                                         db ? dbpart : nullptr, g.N, g.K, l.Kp, g.P, act, c->sigmoid_grad_math);
    int rc = launch_status(c, "pack_dz_kernel");
    if (rc) return rc;
    if (db) {
        partial_rows_sum_kernel<<<(g.K + 7) / 8, 256, 0, st>>>(dbpart, db, g.K, l.db_rows);
        rc = launch_status(c, "partial_rows_sum_kernel");
    }
    return rc;
}

// The contraction itself, from prepared operands.  Returns false in *used (nothing launched) when a
// tensor map cannot be encoded.
static int launch_wgrad_tma(Context* c, const float* dz_hi, const float* dz_lo, const float* xn_hi, const float* xn_lo,
                            float* part, float* dW, const ConvGeom& g, const TmaWgradLayout& l, cudaStream_t st, bool* used) {
    *used = false;
    TmaWgradParams prm;
    {
        const uint64_t dims[5] = {64, (uint64_t)l.Kp / 16, (uint64_t)g.OW, (uint64_t)g.OH, (uint64_t)l.n4};
        const uint64_t str[4] = {256, (uint64_t)l.Kp * 16, (uint64_t)g.OW * l.Kp * 16, (uint64_t)g.P * l.Kp * 16};
        const uint32_t box[5] = {64, 8, (uint32_t)l.bw, (uint32_t)l.bh, 1};
        if (!encode_f32_map(&prm.a_hi, dz_hi, 5, dims, str, box) || !encode_f32_map(&prm.a_lo, dz_lo, 5, dims, str, box))
            return FXB_OK;
    }
    {
        const uint64_t dims[5] = {64, (uint64_t)l.Cp / 16, (uint64_t)l.Wc, (uint64_t)l.Hc, (uint64_t)l.ncls * l.n4};
        const uint64_t str[4] = {256, (uint64_t)l.Cp * 16, (uint64_t)l.Wc * l.Cp * 16, (uint64_t)l.Hc * l.Wc * l.Cp * 16};
        const uint32_t box[5] = {64, (uint32_t)l.Cb / 16, (uint32_t)l.bw, (uint32_t)l.bh, 1};
        if (!encode_f32_map(&prm.b_hi, xn_hi, 5, dims, str, box) || !encode_f32_map(&prm.b_lo, xn_lo, 5, dims, str, box))
            return FXB_OK;
    }
    *used = true;
    prm.tm = l.tm; prm.tn = l.tn; prm.splits = l.splits;
    prm.stages_total = l.stages_total; prm.stages_per_split = l.stages_per_split;
    prm.three_pass = c->math_mode == FXB_MATH_3XTF32 ? 1 : 0;
    prm.drain_group = c->drain_group;
    prm.K = g.K; prm.C = g.C; prm.RS = g.RS; prm.S = g.S;
    prm.Cb = l.Cb; prm.tpt = l.tpt; prm.cblocks = l.cblocks;
    prm.sh = g.sh; prm.sw = g.sw; prm.n4 = l.n4; prm.ncls = l.ncls; prm.bw = l.bw; prm.bh = l.bh;
    prm.dSpg.init((uint32_t)l.spg); prm.dPW.init((uint32_t)l.PWs);
    prm.out = l.splits > 1 ? part : dW;
    prm.split_stride = (int64_t)g.K * g.CRS;
    using Cfg = TmaCfg<128>;
    auto kern = umma_tma_wgrad_kernel<128>;
    static bool attr_set[64] = {};
    if (!attr_set[c->device & 63]) {
        FXB_CUDA_OK(c, cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
        attr_set[c->device & 63] = true;
    }
    const long long items = (long long)l.tm * l.tn * l.splits;
    const int grid = (int)std::min<long long>(items, c->sm_count);
    kern<<<grid, TMA_THREADS, Cfg::SMEM_BYTES, st>>>(prm, c->d_status);
    int rc = launch_status(c, "umma_tma_wgrad_kernel");
    if (rc) return rc;
    if (l.splits > 1) {
        const int64_t n = (int64_t)g.K * g.CRS;
        const int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)c->sm_count * 8);
        splitk_reduce_kernel<float><<<blocks, 256, 0, st>>>(part, dW, n, n, l.splits);
        return launch_status(c, "splitk_reduce");
    }
    return FXB_OK;
}

struct WgradWs { float *dz_hi, *dz_lo, *xn_hi, *xn_lo, *part, *dbpart; };
static WgradWs carve_wgrad_ws(void* ws, const TmaWgradLayout& l, bool with_xn) {
    WgradWs w{};
    char* p = static_cast<char*>(ws);
    w.dz_hi = reinterpret_cast<float*>(p); p += align_up256((size_t)l.dz_floats * 4);
    w.dz_lo = reinterpret_cast<float*>(p); p += align_up256((size_t)l.dz_floats * 4);
    if (with_xn) {
        w.xn_hi = reinterpret_cast<float*>(p); p += align_up256((size_t)l.xn_floats * 4);
        w.xn_lo = reinterpret_cast<float*>(p); p += align_up256((size_t)l.xn_floats * 4);
    }
    w.part = reinterpret_cast<float*>(p); p += align_up256((size_t)l.part_floats * 4);
    w.dbpart = reinterpret_cast<float*>(p);
    return w;
}

// xn_hi / xn_lo: the packed input prepared earlier (by the forward pass), or nullptr: packed here.
static int conv_wgrad_tma(Context* c, const float* X, const float* dY, const float* Yact, float* dW, float* db,
                          const ConvGeom& g, int act, void* ws, size_t ws_bytes, cudaStream_t st, bool* used,
                          const float* xn_hi = nullptr, const float* xn_lo = nullptr) {
    *used = false;
    if (tensor_map_encoder() == nullptr) return FXB_OK;
    const TmaWgradLayout l = tma_wgrad_layout(c, g);
    const bool own_xn = xn_hi == nullptr;
    if (!l.ok || ws == nullptr || (reinterpret_cast<uintptr_t>(ws) & 255) != 0 || ws_bytes < (own_xn ? l.bytes : l.bytes_without_xn))
        return FXB_OK;
    const WgradWs w = carve_wgrad_ws(ws, l, own_xn);
    if (own_xn) { xn_hi = w.xn_hi; xn_lo = w.xn_lo; }
    // probe the tensor maps before anything is launched (the caller falls back to the gather path otherwise)
    {
        TmaWgradParams probe;
        const uint64_t dims[5] = {64, (uint64_t)l.Kp / 16, (uint64_t)g.OW, (uint64_t)g.OH, (uint64_t)l.n4};
        const uint64_t str[4] = {256, (uint64_t)l.Kp * 16, (uint64_t)g.OW * l.Kp * 16, (uint64_t)g.P * l.Kp * 16};
        const uint32_t box[5] = {64, 8, (uint32_t)l.bw, (uint32_t)l.bh, 1};
        const uint64_t dimsb[5] = {64, (uint64_t)l.Cp / 16, (uint64_t)l.Wc, (uint64_t)l.Hc, (uint64_t)l.ncls * l.n4};
        const uint64_t strb[4] = {256, (uint64_t)l.Cp * 16, (uint64_t)l.Wc * l.Cp * 16, (uint64_t)l.Hc * l.Wc * l.Cp * 16};
        const uint32_t boxb[5] = {64, (uint32_t)l.Cb / 16, (uint32_t)l.bw, (uint32_t)l.bh, 1};
        if (!encode_f32_map(&probe.a_hi, w.dz_hi, 5, dims, str, box) || !encode_f32_map(&probe.b_hi, xn_hi, 5, dimsb, strb, boxb))
            return FXB_OK;
    }
    *used = true;
    int rc = launch_pack_dz(c, dY, Yact, w.dz_hi, w.dz_lo, nullptr, nullptr, w.dbpart, db, g, l, act, st);
    if (rc) return rc;
    if (own_xn) {
        rc = launch_pack_xn(c, X, w.xn_hi, w.xn_lo, g, l.Cp, l.Hc, l.Wc, st);
        if (rc) return rc;
    }
    bool launched = false;
    rc = launch_wgrad_tma(c, w.dz_hi, w.dz_lo, xn_hi, xn_lo, w.part, dW, g, l, st, &launched);
    if (rc == FXB_OK && !launched) return fail(c, FXB_ERR_CUDA, "filter gradient: tensor map encoding failed after the probe");
    return rc;
}

template <typename T>
static int conv_wgrad_impl(Context* c, const T* X, const T* dY, const T* Yact, T* dW, T* db, const fxb_conv2d_desc* d,
                           int act, void* ws, size_t ws_bytes, cudaStream_t st) {
    ConvGeom g;
    int rc = make_geom(c, d, g);
    if (rc) return rc;
    FXB_CHECK_ARG(c, X && dY && dW, "Cross correlation got a null buffer");
    FXB_CHECK_ARG(c, act == FXB_ACT_NONE || Yact != nullptr, "Fused activation backward needs the layer output");
    if (c->operand_path == FXB_PATH_AUTO && g.CRS <= SMALLC_K && g.K <= 64) {
        const int64_t npix = (int64_t)g.N * g.P;
        const int blocks = smallc_wgrad_blocks(c, npix);
        if (ws != nullptr && ws_bytes >= smallc_wgrad_bytes(c, npix, sizeof(T))) {
            T* part = static_cast<T*>(ws);
            T* dbpart = db ? part + (size_t)blocks * 64 * SMALLC_K : nullptr;
            if constexpr (sizeof(T) == 4) {
                // The tensor-core form: needs a free im2col column for the bias gradient and 16-byte chunks of
                // four pixels that stay inside one output row.
                const T* ya = act == FXB_ACT_NONE ? nullptr : Yact;
                if (g.CRS < SMALLC_K && g.P % 4 == 0 && g.OW % 4 == 0 && aligned16(dY) && (ya == nullptr || aligned16(ya)) &&
                    (reinterpret_cast<uintptr_t>(ws) & 15) == 0) {
                    const int64_t ntiles = (npix + FLW_BK - 1) / FLW_BK;
                    const int grid = (int)std::min<int64_t>(std::min<int64_t>(blocks, c->sm_count), ntiles);
                    static bool attr_set[64] = {};
                    if (!attr_set[c->device & 63]) {
                        FXB_CUDA_OK(c, cudaFuncSetAttribute(firstlayer_wgrad_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                            FLW_SMEM_BYTES));
                        attr_set[c->device & 63] = true;
                    }
                    firstlayer_wgrad_umma_kernel<<<grid, FLW_THREADS, FLW_SMEM_BYTES, st>>>(X, dY, ya, part, dbpart, g, npix, act,
                                                                                           c->sigmoid_grad_math,
                                                                                           c->math_mode == FXB_MATH_3XTF32 ? 1 : 0,
                                                                                           c->d_status);
                    rc = launch_status(c, "firstlayer_wgrad_umma_kernel");
                    if (rc) return rc;
                    smallc_wgrad_finish_kernel<T><<<64 * SMALLC_K / 32, 256, 0, st>>>(part, dW, g.K, g.CRS, grid);
                    if (db) smallc_db_finish_kernel<T><<<2, 256, 0, st>>>(dbpart, db, g.K, grid);
                    return launch_status(c, "smallc_wgrad_finish_kernel", db ? 2 : 1);
                }
            }
            if constexpr (sizeof(T) == 4)
                smallc_conv_wgrad_f32_kernel<<<blocks, 256, 0, st>>>(X, dY, act == FXB_ACT_NONE ? nullptr : Yact, part, dbpart, g, npix,
                                                                     act, c->sigmoid_grad_math);
            else
                smallc_conv_wgrad_kernel<T><<<blocks, 256, 0, st>>>(X, dY, act == FXB_ACT_NONE ? nullptr : Yact, part, dbpart, g, npix,
                                                                    act, c->sigmoid_grad_math);
            rc = launch_status(c, "smallc_conv_wgrad_kernel");
            if (rc) return rc;
            smallc_wgrad_finish_kernel<T><<<64 * SMALLC_K / 32, 256, 0, st>>>(part, dW, g.K, g.CRS, blocks);
            if (db) smallc_db_finish_kernel<T><<<2, 256, 0, st>>>(dbpart, db, g.K, blocks);
            return launch_status(c, "smallc_wgrad_finish_kernel", db ? 2 : 1);
        }
    }
    if constexpr (sizeof(T) == 4) {
        if (c->operand_path == FXB_PATH_AUTO) {
            bool used = false;
            rc = conv_wgrad_tma(c, reinterpret_cast<const float*>(X), reinterpret_cast<const float*>(dY),
                                reinterpret_cast<const float*>(Yact), reinterpret_cast<float*>(dW), reinterpret_cast<float*>(db),
                                g, act, ws, ws_bytes, st, &used);
            if (rc || used) return rc;
        }
    }
    WgradInputLoader<T> la;
    la.x = X; la.g = g; la.Ktot = g.N * g.P;
    WgradGradLoader<T> lb;
    lb.dy = dY; lb.aux = act == FXB_ACT_NONE ? nullptr : Yact; lb.g = g; lb.Ktot = g.N * g.P;
    lb.act = act; lb.sig_math = c->sigmoid_grad_math;
    lb.vec_ok = (g.P % 4 == 0) && aligned16(dY) && (lb.aux == nullptr || aligned16(lb.aux));
    Problem<T> p;
    p.M = g.CRS; p.N = g.K; p.K = g.N * g.P;
    p.rowsum_b = db;
    p.ws = ws; p.ws_bytes = ws_bytes;
    p.allow_split = true;
    p.out_elems = (int64_t)g.K * g.CRS;
    // dW[ko][crs]: row m = crs inside one "image" of plane CRS, column n = ko with stride CRS.
    auto ow = make_plane_writer<T>(dW, g.CRS, (int64_t)g.K * g.CRS, nullptr, FXB_ACT_NONE, p.M, p.N);
    return launch_contract(c, la, lb, ow, p, st);
}

// ---- whole backward of a conv layer (dW, db, dX) with one operand pass over dY ----------------------
// Packed input of the filter-gradient kernel: [XN hi | XN lo].  0 when the layer does not take the
// tensor-map filter-gradient path.
static size_t conv_packed_bytes(const Context* c, const ConvGeom& g) {
    if (g.CRS <= SMALLC_K || tensor_map_encoder() == nullptr) return 0;
    const TmaWgradLayout l = tma_wgrad_layout(c, g);
    return l.ok ? 2 * align_up256((size_t)l.xn_floats * 4) : 0;
}
static size_t conv_backward_bytes(const Context* c, const ConvGeom& g) {
    const TmaWgradLayout l = tma_wgrad_layout(c, g);
    return l.ok ? align_up256(dgrad_split_bytes(g)) + l.bytes : 0;
}

// Forward pass that also leaves the packed input for the backward pass in `packed` (same values as the
// plain forward).  *packed_written reports whether it did (only the tensor-map path can).
static int conv_fprop_packing(Context* c, const float* X, const float* W, const float* bias, float* Y,
                              const fxb_conv2d_desc* d, int act, void* ws, size_t ws_bytes, void* packed, size_t packed_bytes,
                              int* packed_written, cudaStream_t st, FpropChain* chain = nullptr) {
    if (packed_written) *packed_written = 0;
    ConvGeom g;
    int rc = make_geom(c, d, g);
    if (rc) return rc;
    const size_t need = conv_packed_bytes(c, g);
    if (packed != nullptr && need > 0 && packed_bytes >= need && (reinterpret_cast<uintptr_t>(packed) & 255) == 0 && X && W && Y &&
        act >= FXB_ACT_NONE && act <= FXB_ACT_TANH && c->operand_path == FXB_PATH_AUTO && ws != nullptr &&
        (reinterpret_cast<uintptr_t>(ws) & 255) == 0 && ws_bytes >= fprop_split_bytes(c, g)) {
        const TmaWgradLayout l = tma_wgrad_layout(c, g);
        float* xn_hi = static_cast<float*>(packed);
        float* xn_lo = reinterpret_cast<float*>(static_cast<char*>(packed) + align_up256((size_t)l.xn_floats * 4));
        bool used = false;
        rc = conv_fprop_tma(c, X, W, bias, Y, g, act, ws, st, &used, FPROP_ALL, xn_hi, xn_lo, l.Cp, chain);
        if (rc) return rc;
        if (used) {
            if (packed_written) *packed_written = 1;
            return FXB_OK;
        }
    }
    return conv_fprop_impl<float>(c, X, W, bias, Y, d, act, ws, ws_bytes, st, FPROP_ALL, chain);
}

// The chained forward: optional input slabs (written by the previous layer's call) and optional emission of the
// next layer's slabs.  Anything that does not fit is ignored (the call then behaves like the packing forward).
static int conv_fprop_chain(Context* c, const float* X, const float* W, const float* bias, float* Y, const fxb_conv2d_desc* d,
                            int act, void* ws, size_t ws_bytes, void* packed, size_t packed_bytes, int* packed_written,
                            const void* in_slabs, const fxb_conv2d_desc* next, void* out_slabs, size_t out_slab_bytes,
                            int* out_written, cudaStream_t st) {
    if (out_written) *out_written = 0;
    ConvGeom g;
    int rc = make_geom(c, d, g);
    if (rc) return rc;
    FpropChain ch;
    if (in_slabs != nullptr && (reinterpret_cast<uintptr_t>(in_slabs) & 255) == 0 && conv_input_slab_bytes(g) > 0) {
        const TmaFpropLayout l = tma_fprop_layout(g);
        ch.in_hi = static_cast<const float*>(in_slabs);
        ch.in_lo = reinterpret_cast<const float*>(static_cast<const char*>(in_slabs) + align_up256((size_t)l.image_floats * 4));
    }
    if (next != nullptr && out_slabs != nullptr) {
        ConvGeom g2;
        rc = make_geom(c, next, g2);
        if (rc) return rc;
        FXB_CHECK_ARG(c, g2.N == g.N && g2.C == g.K && g2.H == g.OH && g2.W == g.OW,
                      "Conv2D chain: the next layer's input shape is not this layer's output shape");
        const size_t need = conv_input_slab_bytes(g2);
        if (need > 0 && out_slab_bytes >= need && (reinterpret_cast<uintptr_t>(out_slabs) & 255) == 0 &&
            c->operand_path == FXB_PATH_AUTO)
            ch.emit = make_slab_emit(g2, out_slabs);
    }
    rc = conv_fprop_packing(c, X, W, bias, Y, d, act, ws, ws_bytes, packed, packed_bytes, packed_written, st, &ch);
    if (rc == FXB_OK && out_written) *out_written = ch.emitted ? 1 : 0;
    return rc;
}

template <typename T>
static int conv_backward_impl(Context* c, const T* X, const T* dY, const T* Yact, const T* W, T* dX, T* dW, T* db,
                              const fxb_conv2d_desc* d, int act, void* ws, size_t ws_bytes, const void* packed,
                              cudaStream_t st) {
    ConvGeom g;
    int rc = make_geom(c, d, g);
    if (rc) return rc;
    FXB_CHECK_ARG(c, X && dY && W && dW, "Conv2d backward got a null buffer");
    FXB_CHECK_ARG(c, act == FXB_ACT_NONE || Yact != nullptr, "Fused activation backward needs the layer output");
    if constexpr (sizeof(T) == 4) {
        const TmaWgradLayout l = tma_wgrad_layout(c, g);
        const bool fused = c->operand_path == FXB_PATH_AUTO && dX != nullptr && g.CRS > SMALLC_K && l.ok && tensor_map_encoder() != nullptr &&
                           ws != nullptr && (reinterpret_cast<uintptr_t>(ws) & 255) == 0 && ws_bytes >= conv_backward_bytes(c, g);
        if (fused) {
            // region 1: the input-gradient operands (dZ slabs, filter); region 2: the filter-gradient operands
            const size_t r1 = align_up256(dgrad_split_bytes(g));
            void* ws2 = static_cast<char*>(ws) + r1;
            const int K4 = (g.K + 3) / 4;
            const int bn = tile_cols(g.C);
            const SplitWs sw = carve_split_ws(ws, (int64_t)g.N * K4 * g.P * 4, (int64_t)round_up(g.C, bn) * g.RS * K4 * 4);
            const float* xn_hi = static_cast<const float*>(packed);
            const float* xn_lo = packed ? reinterpret_cast<const float*>(static_cast<const char*>(packed) + align_up256((size_t)l.xn_floats * 4))
                                        : nullptr;
            const bool own_xn = packed == nullptr;
            const WgradWs w = carve_wgrad_ws(ws2, l, own_xn);
            if (own_xn) { xn_hi = w.xn_hi; xn_lo = w.xn_lo; }
            rc = launch_pack_dz(c, dY, Yact, w.dz_hi, w.dz_lo, sw.a_hi, sw.a_lo, w.dbpart, db, g, l, act, st);
            if (rc) return rc;
            if (own_xn) {
                rc = launch_pack_xn(c, X, w.xn_hi, w.xn_lo, g, l.Cp, l.Hc, l.Wc, st);
                if (rc) return rc;
            }
            bool launched = false;
            rc = launch_wgrad_tma(c, w.dz_hi, w.dz_lo, xn_hi, xn_lo, w.part, dW, g, l, st, &launched);
            if (rc) return rc;
            if (!launched) {  // no tensor map for this shape: the general filter-gradient path (region 2 is free again)
                rc = conv_wgrad_impl<float>(c, X, dY, Yact, dW, nullptr, d, act, ws2, ws_bytes - r1, st);
                if (rc) return rc;
            }
            bool used = false;
            rc = conv_dgrad_tma(c, dY, Yact, W, dX, g, act, ws, st, &used, true);
            if (rc || used) return rc;
            return conv_dgrad_impl<float>(c, dY, Yact, W, dX, d, act, ws, ws_bytes, st);
        }
    }
    rc = conv_wgrad_impl<T>(c, X, dY, Yact, dW, db, d, act, ws, ws_bytes, st);
    if (rc || dX == nullptr) return rc;
    return conv_dgrad_impl<T>(c, dY, Yact, W, dX, d, act, ws, ws_bytes, st);
}

// Batch rows per partial-sum chunk of the skinny dW kernel: small enough for about two CTAs per SM, a power of
// two between 8 and SKINNY_ROWS.
static int skinny_rows_per_chunk(const Context* c, int64_t B, int64_t in) {
    const int64_t colblocks = (in + 255) / 256;
    const int64_t want_chunks = std::max<int64_t>(1, (2 * (int64_t)c->sm_count + colblocks - 1) / colblocks);
    int rows = SKINNY_ROWS;
    while (rows > 8 && (B + rows - 1) / rows < want_chunks) rows >>= 1;
    return rows;
}
template <typename T>
static size_t skinny_bwd_bytes(const Context* c, int64_t B, int64_t in, int64_t out) {
    const int rows = skinny_rows_per_chunk(c, B, in);
    const int64_t chunks = (B + rows - 1) / rows;
    return chunks > 1 ? (size_t)(chunks * out * in + chunks * out) * sizeof(T) : 0;
}

template <typename T>
static int linear_fwd_impl(Context* c, const T* X, const T* W, const T* bias, T* Y, int64_t B, int64_t in, int64_t out,
                           int act, cudaStream_t st, void* ws = nullptr, size_t ws_bytes = 0) {
    FXB_CHECK_ARG(c, B >= 0 && in > 0 && out > 0, "Linear layer sizes must be positive");
    if (out <= SKINNY_MAXO && fits_i32(B) && fits_i32(in)) {
        // a few output features: one warp per batch row on the CUDA cores (memory-bound)
        if (B == 0) return FXB_OK;
        FXB_CHECK_ARG(c, X && W && Y, "Matrix multiplication got a null buffer");
        FXB_CHECK_ARG(c, act >= FXB_ACT_NONE && act <= FXB_ACT_TANH, "Unknown activation code");
        // four rows per block once that still gives two blocks per SM; one row per block for small batches
        if (B >= (int64_t)8 * c->sm_count)
            skinny_linear_fwd_kernel<T, 4><<<(unsigned)((B + 3) / 4), 256, 0, st>>>(X, W, bias, Y, (int)B, (int)in, (int)out, act);
        else
            skinny_linear_fwd_kernel<T, 1><<<(unsigned)B, 256, 0, st>>>(X, W, bias, Y, (int)B, (int)in, (int)out, act);
        return launch_status(c, "skinny_linear_fwd_kernel");
    }
    // (the workspace only serves the tensor-map path: this product never splits K)
    const bool tma = sizeof(T) == 4 && ws != nullptr && tma_gemm_wanted(c, B, out, in) && ws_bytes >= tma_gemm_bytes(B, out, in);
    return gemm_impl<T>(c, 0, 1, B, out, in, X, in, W, in, Y, out, bias, act, nullptr, 0, nullptr, tma ? ws : nullptr,
                        tma ? ws_bytes : 0, st);
}

template <typename T>
static int linear_bwd_impl(Context* c, const T* X, const T* W, const T* Y, const T* dY, T* dX, T* dW, T* db, int64_t B,
                           int64_t in, int64_t out, int act, void* ws, size_t ws_bytes, cudaStream_t st) {
    FXB_CHECK_ARG(c, B > 0 && in > 0 && out > 0, "Linear layer sizes must be positive");
    FXB_CHECK_ARG(c, X && W && dY && dW, "Linear backward got a null buffer");
    FXB_CHECK_ARG(c, act == FXB_ACT_NONE || Y != nullptr, "Fused activation backward needs the layer output");
    const T* aux = act == FXB_ACT_NONE ? nullptr : Y;
    // grid limits of the three kernels: chunks of at least 8 rows and blocks of 256 columns in grid.y (<= 65535)
    if (out <= SKINNY_MAXO && fits_i32(B) && fits_i32(in) && B <= 65535 * (int64_t)8 && in <= 65535 * (int64_t)256) {
        const int rpc = skinny_rows_per_chunk(c, B, in);
        const int chunks = (int)((B + rpc - 1) / rpc);
        const size_t need = skinny_bwd_bytes<T>(c, B, in, out);
        if (chunks == 1 || (ws != nullptr && ws_bytes >= need)) {
            T* part = chunks == 1 ? dW : static_cast<T*>(ws);
            T* dbpart = db == nullptr ? nullptr : (chunks == 1 ? db : part + (size_t)chunks * out * in);
            dim3 grid((unsigned)((in + 255) / 256), (unsigned)chunks);
            skinny_linear_dw_kernel<T><<<grid, 256, 0, st>>>(X, dY, aux, part, dbpart, (int)B, (int)in, (int)out, act,
                                                             c->sigmoid_grad_math, rpc);
            int rc = launch_status(c, "skinny_linear_dw_kernel");
            if (rc) return rc;
            if (chunks > 1) {
                const int64_t n = out * in;
                const int blocks = (int)std::min<int64_t>((n + 255) / 256, (int64_t)c->sm_count * 8);
                splitk_reduce_kernel<T><<<blocks, 256, 0, st>>>(part, dW, n, n, chunks);
                if (db) splitk_reduce_kernel<T><<<1, 256, 0, st>>>(dbpart, db, out, out, chunks);
                rc = launch_status(c, "splitk_reduce", db ? 2 : 1);
                if (rc) return rc;
            }
            if (dX) {
                // rows per block: as many as leave about four blocks per SM (at most SKINNY_DX_ROWS)
                const int64_t slices = (in + 255) / 256;
                int rows = (int)std::max<int64_t>(1, std::min<int64_t>(SKINNY_DX_ROWS, B * slices / ((int64_t)c->sm_count * 4)));
                dim3 gx((unsigned)((B + rows - 1) / rows), (unsigned)slices);
                skinny_linear_dx_kernel<T><<<gx, 256, 0, st>>>(dY, aux, W, dX, (int)B, (int)in, (int)out, act, c->sigmoid_grad_math,
                                                               rows);
                rc = launch_status(c, "skinny_linear_dx_kernel");
            }
            return rc;
        }
    }
    // dW[out,in] = dZ^T . X   (A(m=o,k=b) = dZ[b,o], B(n=i,k=b) = X[b,i]); db = row sums of A.
    int rc = gemm_impl<T>(c, 1, 0, out, in, B, dY, out, X, in, dW, in, nullptr, FXB_ACT_NONE, aux, act, db, ws, ws_bytes, st);
    if (rc) return rc;
    // dX[B,in] = dZ . W   (A(m=b,k=o) = dZ[b,o], B(n=i,k=o) = W[o,i])
    //   (the workspace is free again: the dW call's kernels precede this one on the stream; without the tensor-map
    //    path this product never splits K, as before)
    if (dX) {
        const bool tma = sizeof(T) == 4 && tma_gemm_wanted(c, B, in, out) && ws_bytes >= tma_gemm_bytes(B, in, out);
        rc = gemm_impl<T>(c, 0, 0, B, in, out, dY, out, W, in, dX, in, nullptr, FXB_ACT_NONE, aux, act, nullptr, tma ? ws : nullptr,
                          tma ? ws_bytes : 0, st);
    }
    return rc;
}

}  // namespace fxb

using namespace fxb;
#define CTX(h) reinterpret_cast<fxb::Context*>(h)
#define ST(s) static_cast<cudaStream_t>(s)
#define NEED_HANDLE(h) \
    if ((h) == nullptr) return fxb::fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle")

#define FXB_CONTRACT_API(SUF, T)                                                                                        \
    extern "C" int fxb_matmul_##SUF(fxb_handle_t h, const T* A, const T* B, T* C, int64_t M, int64_t N, int64_t K,      \
                                    fxb_stream_t s) {                                                                   \
        NEED_HANDLE(h);                                                                                                 \
        return gemm_impl<T>(CTX(h), 0, 0, M, N, K, A, K, B, N, C, N, nullptr, FXB_ACT_NONE, nullptr, 0, nullptr,        \
                            nullptr, 0, ST(s));                                                                         \
    }                                                                                                                   \
    extern "C" int fxb_gemm_##SUF(fxb_handle_t h, int ta, int tb, int64_t M, int64_t N, int64_t K, const T* A,          \
                                  int64_t lda, const T* B, int64_t ldb, T* C, int64_t ldc, const T* bias, int act,      \
                                  void* ws, size_t wsb, fxb_stream_t s) {                                               \
        NEED_HANDLE(h);                                                                                                 \
        return gemm_impl<T>(CTX(h), ta, tb, M, N, K, A, lda, B, ldb, C, ldc, bias, act, nullptr, 0, nullptr, ws, wsb,   \
                            ST(s));                                                                                     \
    }                                                                                                                   \
    extern "C" int fxb_linear_fwd_##SUF(fxb_handle_t h, const T* X, const T* W, const T* bias, T* Y, int64_t B,         \
                                        int64_t in, int64_t out, int act, fxb_stream_t s) {                             \
        NEED_HANDLE(h);                                                                                                 \
        return linear_fwd_impl<T>(CTX(h), X, W, bias, Y, B, in, out, act, ST(s));                                       \
    }                                                                                                                   \
    extern "C" int fxb_linear_fwd_ws_##SUF(fxb_handle_t h, const T* X, const T* W, const T* bias, T* Y, int64_t B,      \
                                           int64_t in, int64_t out, int act, void* ws, size_t wsb, fxb_stream_t s) {    \
        NEED_HANDLE(h);                                                                                                 \
        return linear_fwd_impl<T>(CTX(h), X, W, bias, Y, B, in, out, act, ST(s), ws, wsb);                              \
    }                                                                                                                   \
    extern "C" int fxb_linear_bwd_##SUF(fxb_handle_t h, const T* X, const T* W, const T* Y, const T* dY, T* dX, T* dW,  \
                                        T* db, int64_t B, int64_t in, int64_t out, int act, void* ws, size_t wsb,       \
                                        fxb_stream_t s) {                                                               \
        NEED_HANDLE(h);                                                                                                 \
        return linear_bwd_impl<T>(CTX(h), X, W, Y, dY, dX, dW, db, B, in, out, act, ws, wsb, ST(s));                    \
    }                                                                                                                   \
    extern "C" int fxb_conv2d_forward_##SUF(fxb_handle_t h, const T* X, const T* W, T* Y, const fxb_conv2d_desc* d,     \
                                            void* ws, size_t wsb, fxb_stream_t s) {                                     \
        NEED_HANDLE(h);                                                                                                 \
        return conv_fprop_impl<T>(CTX(h), X, W, nullptr, Y, d, FXB_ACT_NONE, ws, wsb, ST(s));                           \
    }                                                                                                                   \
    extern "C" int fxb_conv2d_bias_act_fwd_##SUF(fxb_handle_t h, const T* X, const T* W, const T* bias, T* Y,           \
                                                 const fxb_conv2d_desc* d, int act, void* ws, size_t wsb,               \
                                                 fxb_stream_t s) {                                                      \
        NEED_HANDLE(h);                                                                                                 \
        return conv_fprop_impl<T>(CTX(h), X, W, bias, Y, d, act, ws, wsb, ST(s));                                       \
    }                                                                                                                   \
    extern "C" int fxb_deconv2d_##SUF(fxb_handle_t h, const T* dY, const T* W, T* dX, const fxb_conv2d_desc* d,         \
                                      void* ws, size_t wsb, fxb_stream_t s) {                                           \
        NEED_HANDLE(h);                                                                                                 \
        return conv_dgrad_impl<T>(CTX(h), dY, nullptr, W, dX, d, FXB_ACT_NONE, ws, wsb, ST(s));                         \
    }                                                                                                                   \
    extern "C" int fxb_conv2d_dgrad_act_##SUF(fxb_handle_t h, const T* dY, const T* Y, const T* W, T* dX,               \
                                              const fxb_conv2d_desc* d, int act, void* ws, size_t wsb,                  \
                                              fxb_stream_t s) {                                                         \
        NEED_HANDLE(h);                                                                                                 \
        return conv_dgrad_impl<T>(CTX(h), dY, Y, W, dX, d, act, ws, wsb, ST(s));                                        \
    }                                                                                                                   \
    extern "C" int fxb_cross_correlation2d_##SUF(fxb_handle_t h, const T* X, const T* dY, T* dW,                        \
                                                 const fxb_conv2d_desc* d, void* ws, size_t wsb, fxb_stream_t s) {      \
        NEED_HANDLE(h);                                                                                                 \
        return conv_wgrad_impl<T>(CTX(h), X, dY, nullptr, dW, nullptr, d, FXB_ACT_NONE, ws, wsb, ST(s));                \
    }                                                                                                                   \
    extern "C" int fxb_conv2d_wgrad_bias_act_##SUF(fxb_handle_t h, const T* X, const T* dY, const T* Y, T* dW, T* db,   \
                                                   const fxb_conv2d_desc* d, int act, void* ws, size_t wsb,             \
                                                   fxb_stream_t s) {                                                    \
        NEED_HANDLE(h);                                                                                                 \
        return conv_wgrad_impl<T>(CTX(h), X, dY, Y, dW, db, d, act, ws, wsb, ST(s));                                    \
    }

FXB_CONTRACT_API(f32, float)
FXB_CONTRACT_API(f64, double)

extern "C" int fxb_conv2d_backward_f32(fxb_handle_t h, const float* X, const float* dY, const float* Y, const float* W, float* dX,
                                       float* dW, float* db, const fxb_conv2d_desc* d, int act, void* ws, size_t wsb,
                                       const void* packed_input, fxb_stream_t s) {
    NEED_HANDLE(h);
    return conv_backward_impl<float>(CTX(h), X, dY, Y, W, dX, dW, db, d, act, ws, wsb, packed_input, ST(s));
}
extern "C" int fxb_conv2d_backward_f64(fxb_handle_t h, const double* X, const double* dY, const double* Y, const double* W,
                                       double* dX, double* dW, double* db, const fxb_conv2d_desc* d, int act, void* ws,
                                       size_t wsb, const void* packed_input, fxb_stream_t s) {
    NEED_HANDLE(h);
    (void)packed_input;  // f64 has no packed operands
    return conv_backward_impl<double>(CTX(h), X, dY, Y, W, dX, dW, db, d, act, ws, wsb, nullptr, ST(s));
}
extern "C" int fxb_conv2d_bias_act_fwd_packing_f32(fxb_handle_t h, const float* X, const float* W, const float* bias, float* Y,
                                                   const fxb_conv2d_desc* d, int act, void* ws, size_t wsb, void* packed_input,
                                                   size_t packed_bytes, int* packed_written, fxb_stream_t s) {
    NEED_HANDLE(h);
    return conv_fprop_packing(CTX(h), X, W, bias, Y, d, act, ws, wsb, packed_input, packed_bytes, packed_written, ST(s));
}
extern "C" int fxb_conv2d_bias_act_fwd_chain_f32(fxb_handle_t h, const float* X, const float* W, const float* bias, float* Y,
                                                 const fxb_conv2d_desc* d, int act, void* ws, size_t wsb, void* packed_input,
                                                 size_t packed_bytes, int* packed_written, const void* input_slabs,
                                                 const fxb_conv2d_desc* next, void* output_slabs, size_t output_slab_bytes,
                                                 int* output_slabs_written, fxb_stream_t s) {
    NEED_HANDLE(h);
    return conv_fprop_chain(CTX(h), X, W, bias, Y, d, act, ws, wsb, packed_input, packed_bytes, packed_written, input_slabs, next,
                            output_slabs, output_slab_bytes, output_slabs_written, ST(s));
}
extern "C" size_t fxb_conv2d_input_slab_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem) {
    if (!h || !d || elem != 4) return 0;
    ConvGeom g;
    if (make_geom(CTX(h), d, g) != FXB_OK) return 0;
    return conv_input_slab_bytes(g);
}
extern "C" size_t fxb_conv2d_packed_input_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem) {
    if (!h || !d || elem != 4) return 0;
    ConvGeom g;
    if (make_geom(CTX(h), d, g) != FXB_OK) return 0;
    return conv_packed_bytes(CTX(h), g);
}
extern "C" size_t fxb_conv2d_backward_workspace_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem) {
    if (!h || !d) return 0;
    ConvGeom g;
    if (make_geom(CTX(h), d, g) != FXB_OK) return 0;
    size_t need = std::max(fxb_conv2d_wgrad_workspace_bytes(h, d, elem), fxb_conv2d_dgrad_workspace_bytes(h, d, elem));
    if (elem == 4) need = std::max(need, conv_backward_bytes(CTX(h), g));
    return need;
}

extern "C" size_t fxb_gemm_workspace_bytes(fxb_handle_t h, int64_t M, int64_t N, int64_t K, size_t elem) {
    if (!h || M <= 0 || N <= 0 || K <= 0) return 0;
    size_t need = split_ws_upper(CTX(h), M, N, K, M * N, 0, 0, elem);
    if (elem == 4 && tma_gemm_wanted(CTX(h), M, N, K)) need = std::max(need, tma_gemm_bytes(M, N, K));
    return need;
}
extern "C" size_t fxb_linear_fwd_workspace_bytes(fxb_handle_t h, int64_t B, int64_t in, int64_t out, size_t elem) {
    if (!h || B <= 0 || in <= 0 || out <= 0) return 0;
    return (elem == 4 && out > SKINNY_MAXO && tma_gemm_wanted(CTX(h), B, out, in)) ? tma_gemm_bytes(B, out, in) : 0;
}
extern "C" size_t fxb_linear_bwd_workspace_bytes(fxb_handle_t h, int64_t B, int64_t in, int64_t out, size_t elem) {
    if (!h || B <= 0 || in <= 0 || out <= 0) return 0;
    size_t need = split_ws_upper(CTX(h), out, in, B, out * in, (int)out, 0, elem);
    if (elem == 4 && out > SKINNY_MAXO) {
        if (tma_gemm_wanted(CTX(h), out, in, B)) need = std::max(need, tma_gemm_bytes(out, in, B));
        if (tma_gemm_wanted(CTX(h), B, in, out)) need = std::max(need, tma_gemm_bytes(B, in, out));
    }
    if (out <= SKINNY_MAXO) need = std::max(need, elem == 8 ? skinny_bwd_bytes<double>(CTX(h), B, in, out) : skinny_bwd_bytes<float>(CTX(h), B, in, out));
    return need;
}
extern "C" int fxb_conv2d_fprop_prepass_f32(fxb_handle_t h, const float* X, const float* W, const fxb_conv2d_desc* d,
                                            void* ws, size_t ws_bytes, fxb_stream_t s) {
    NEED_HANDLE(h);
    Context* c = CTX(h);
    if (c->operand_path != FXB_PATH_AUTO || ws == nullptr)
        return fail(c, FXB_ERR_INVALID_ARGUMENT, "the operand pre-pass needs FXB_PATH_AUTO and a workspace");
    // the output pointer is not touched when the call stops before the contraction
    return conv_fprop_impl<float>(c, X, W, nullptr, reinterpret_cast<float*>(ws), d, FXB_ACT_NONE, ws, ws_bytes, ST(s),
                                  FPROP_PREPASS_ONLY);
}
extern "C" int fxb_conv2d_fprop_main_f32(fxb_handle_t h, const float* bias, float* Y, const fxb_conv2d_desc* d, int act,
                                         void* ws, size_t ws_bytes, fxb_stream_t s) {
    NEED_HANDLE(h);
    Context* c = CTX(h);
    if (c->operand_path != FXB_PATH_AUTO || ws == nullptr)
        return fail(c, FXB_ERR_INVALID_ARGUMENT, "the contraction-only call needs FXB_PATH_AUTO and the pre-pass workspace");
    // X and W are not read: the operands come from the workspace the pre-pass filled
    return conv_fprop_impl<float>(c, reinterpret_cast<const float*>(ws), reinterpret_cast<const float*>(ws), bias, Y, d, act, ws,
                                  ws_bytes, ST(s), FPROP_MAIN_ONLY);
}
extern "C" size_t fxb_conv2d_fprop_workspace_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem) {
    if (!h || !d || elem != 4) return 0;
    ConvGeom g;
    if (make_geom(CTX(h), d, g) != FXB_OK) return 0;
    return fprop_split_bytes(CTX(h), g);
}
extern "C" size_t fxb_conv2d_dgrad_workspace_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem) {
    if (!h || !d || elem != 4) return 0;
    ConvGeom g;
    if (make_geom(CTX(h), d, g) != FXB_OK) return 0;
    return dgrad_split_bytes(g);
}
extern "C" size_t fxb_conv2d_wgrad_workspace_bytes(fxb_handle_t h, const fxb_conv2d_desc* d, size_t elem) {
    if (!h || !d) return 0;
    ConvGeom g;
    if (make_geom(CTX(h), d, g) != FXB_OK) return 0;
    size_t need = split_ws_upper(CTX(h), g.CRS, g.K, (int64_t)g.N * g.P, (int64_t)g.K * g.CRS, 0, g.K, elem);
    if (elem == 4) {
        const TmaWgradLayout l = tma_wgrad_layout(CTX(h), g);
        if (l.ok) need = std::max(need, l.bytes);
    }
    if (g.CRS <= SMALLC_K && g.K <= 64) need = std::max(need, smallc_wgrad_bytes(CTX(h), (int64_t)g.N * g.P, elem));
    return need;
}
