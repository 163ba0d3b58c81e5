// HBM-streaming kernels of the C ABI: activations forward/backward, elementwise add / mul /
// axpby / masks, bias add, sum reductions over arbitrary axes (two-stage, deterministic), the
// fused softmax cross-entropy and the fused optimizer steps.
// All of them are bandwidth bound: 128-bit loads and stores, several independent vectors in
// flight per thread, grids sized in multiples of the SM count.
#include "fxb_common.cuh"

#include <algorithm>
#include <cmath>
#include <vector>

namespace fxb {

constexpr int EW_THREADS = 256;
constexpr int EW_UNROLL = 4;

template <typename T> struct VecOf;                       // 16-byte vectors
template <> struct VecOf<float> { using type = float4; static constexpr int N = 4; };
template <> struct VecOf<double> { using type = double2; static constexpr int N = 2; };

template <typename T> __device__ __forceinline__ void vload(const T* p, T (&v)[VecOf<T>::N]);
template <> __device__ __forceinline__ void vload<float>(const float* p, float (&v)[4]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
template <> __device__ __forceinline__ void vload<double>(const double* p, double (&v)[2]) {
    const double2 x = *reinterpret_cast<const double2*>(p);
    v[0] = x.x; v[1] = x.y;
}
template <typename T> __device__ __forceinline__ void vstore(T* p, const T (&v)[VecOf<T>::N]);
template <> __device__ __forceinline__ void vstore<float>(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void vstore<double>(double* p, const double (&v)[2]) {
    *reinterpret_cast<double2*>(p) = make_double2(v[0], v[1]);
}

// out[i] = f(a[i], b[i]); b may be unused (NIN == 1).  Vector body + scalar tail.
template <typename T, int NIN, class F>
__global__ void __launch_bounds__(EW_THREADS) elementwise_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                                                 T* __restrict__ out, int64_t n, int vec_ok, F f) {
    constexpr int V = VecOf<T>::N;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t nthreads = (int64_t)gridDim.x * blockDim.x;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t nvec = n / V;
        int64_t i = tid;
        for (; i + (EW_UNROLL - 1) * nthreads < nvec; i += EW_UNROLL * nthreads) {
            T va[EW_UNROLL][V], vb[EW_UNROLL][V];
#pragma unroll
            for (int u = 0; u < EW_UNROLL; ++u) {
                vload<T>(a + (i + u * nthreads) * V, va[u]);
                if (NIN == 2) vload<T>(b + (i + u * nthreads) * V, vb[u]);
            }
#pragma unroll
            for (int u = 0; u < EW_UNROLL; ++u) {
                T r[V];
#pragma unroll
                for (int e = 0; e < V; ++e) r[e] = f(va[u][e], NIN == 2 ? vb[u][e] : T(0));
                vstore<T>(out + (i + u * nthreads) * V, r);
            }
        }
        for (; i < nvec; i += nthreads) {
            T va[V], vb[V], r[V];
            vload<T>(a + i * V, va);
            if (NIN == 2) vload<T>(b + i * V, vb);
#pragma unroll
            for (int e = 0; e < V; ++e) r[e] = f(va[e], NIN == 2 ? vb[e] : T(0));
            vstore<T>(out + i * V, r);
        }
        done = nvec * V;
    }
    for (int64_t i = done + tid; i < n; i += nthreads) out[i] = f(a[i], NIN == 2 ? b[i] : T(0));
}

static int ew_grid(const Context* c, int64_t n, int vec) {
    const int64_t per_block = (int64_t)EW_THREADS * vec * EW_UNROLL;
    const int64_t want = (n + per_block - 1) / per_block;
    const int64_t cap = (int64_t)c->sm_count * 16;
    return (int)std::max<int64_t>(1, std::min(want, cap));
}

template <typename T, int NIN, class F>
static int launch_ew(Context* c, const T* a, const T* b, T* out, int64_t n, F f, cudaStream_t st, const char* what) {
    FXB_CHECK_ARG(c, n >= 0, "negative element count");
    if (n == 0) return FXB_OK;
    FXB_CHECK_ARG(c, a != nullptr && out != nullptr && (NIN == 1 || b != nullptr), std::string(what) + ": null buffer");
    auto al = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    const int vec_ok = al(a) && al(out) && (NIN == 1 || al(b));
    elementwise_kernel<T, NIN, F><<<ew_grid(c, n, VecOf<T>::N), EW_THREADS, 0, st>>>(a, b, out, n, vec_ok, f);
    return launch_status(c, what);
}

template <typename T> struct ActFwdF { int act; __device__ T operator()(T x, T) const { return act_apply_full<T>(x, act); } };
template <typename T> struct ActBwdF {
    int act, sig;
    __device__ T operator()(T dy, T aux) const { return dy * act_grad_factor<T>(aux, act, sig); }
};
template <typename T> struct AddF { __device__ T operator()(T a, T b) const { return a + b; } };
template <typename T> struct MulF { __device__ T operator()(T a, T b) const { return a * b; } };
template <typename T> struct AxpbyF { T al, be; __device__ T operator()(T x, T y) const { return al * x + be * y; } };
template <typename T> struct ScaleF { T al; __device__ T operator()(T x, T) const { return al * x; } };
template <typename T> struct GreaterF { T s; __device__ T operator()(T x, T) const { return x > s ? T(1) : T(0); } };

// y[o, ch, p] += bias[ch]
template <typename T>
__global__ void __launch_bounds__(EW_THREADS) bias_add_kernel(T* __restrict__ y, const T* __restrict__ bias, int64_t n,
                                                              FastDiv dplane, int channels) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const uint32_t q = dplane.div((uint32_t)i);
        y[i] += __ldg(bias + (q % (uint32_t)channels));
    }
}

// ------------------------------------------------------------------------------------------
// Sum over axes.  The host collapses the shape into [KB][R0][K0][R1][K1] (R* reduced, K* kept,
// any of them 1) and picks one of two stage-one kernels; both write partial sums
// part[p][out_index] that stage two adds in order p = 0..parts-1.
struct ReduceGeom {
    int64_t KB, R0, K0, R1, K1;
    int parts;
    int64_t outputs;  // KB*K0*K1
};

template <typename T>
__device__ __forceinline__ T block_sum(T v, T* smem) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    T r = T(0);
    if (threadIdx.x == 0) {
        const int nw = blockDim.x >> 5;
        for (int w = 0; w < nw; ++w) r += smem[w];
    }
    return r;  // valid in thread 0
}

// Inner axis reduced (K1 == 1): one CTA sums part p of output (kb,k0): the flattened (r0,r1)
// range [p*len, (p+1)*len), read as contiguous runs of R1 elements.  Index arithmetic is 32-bit
// with multiply-shift division (the host guarantees R0*R1 < 2^31); four independent 16-byte
// loads are in flight per thread.
template <typename T>
__global__ void __launch_bounds__(256) reduce_inner_kernel(const T* __restrict__ x, T* __restrict__ part, ReduceGeom g,
                                                           FastDiv dk0, FastDiv drun, int vec_ok) {
    __shared__ T red[32];
    constexpr int V = VecOf<T>::N;
    const uint32_t o = blockIdx.x;  // output index kb*K0 + k0
    const int p = blockIdx.y;
    uint32_t kb, k0;
    dk0.divmod(o, kb, k0);
    const uint32_t total = (uint32_t)(g.R0 * g.R1);
    const uint32_t len = (total + g.parts - 1) / g.parts;
    const uint32_t e0 = (uint32_t)p * len;
    const uint32_t e1 = e0 + len < total ? e0 + len : total;
    const int64_t run_stride = g.K0 * g.R1;                       // distance between consecutive r0 runs
    const T* base = x + ((int64_t)kb * g.R0 * g.K0 + k0) * g.R1;  // element (r0=0, r1=0) of this output
    T acc[4] = {T(0), T(0), T(0), T(0)};
    if (e0 < e1) {
        if (vec_ok) {
            // R1 % V == 0 and aligned base: runs are whole vectors; drun divides by R1/V
            const uint32_t v0 = e0 / V, v1 = (e1 + V - 1) / V;
            const bool ragged = (e0 % V) != 0 || (e1 % V) != 0;
            uint32_t vi = v0 + threadIdx.x;
            for (; vi + 3 * 256 < v1; vi += 4 * 256) {
                T v[4][V];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    uint32_t r0, rv;
                    drun.divmod(vi + u * 256, r0, rv);
                    vload<T>(base + (int64_t)r0 * run_stride + rv * V, v[u]);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int e = 0; e < V; ++e) {
                        const uint32_t ge = (vi + u * 256) * V + e;
                        if (!ragged || (ge >= e0 && ge < e1)) acc[u] += v[u][e];
                    }
            }
            for (; vi < v1; vi += 256) {
                uint32_t r0, rv;
                drun.divmod(vi, r0, rv);
                T v[V];
                vload<T>(base + (int64_t)r0 * run_stride + rv * V, v);
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    const uint32_t ge = vi * V + e;
                    if (ge >= e0 && ge < e1) acc[0] += v[e];
                }
            }
        } else {
            // drun divides by R1
            int u = 0;
            for (uint32_t e = e0 + threadIdx.x; e < e1; e += 256, u = (u + 1) & 3) {
                uint32_t r0, r1;
                drun.divmod(e, r0, r1);
                acc[u] += base[(int64_t)r0 * run_stride + r1];
            }
        }
    }
    const T s = block_sum<T>((acc[0] + acc[1]) + (acc[2] + acc[3]), red);
    if (threadIdx.x == 0) part[(int64_t)p * g.outputs + o] = s;
}

// Inner axis kept (K1 > 1): CTA = 32 column groups (one vector each) x 8 row lanes; it sums
// part p of the rows (flattened r0,r1) for one (kb,k0) and one tile of 32*V columns.  Four
// independent row loads are in flight per thread.
template <typename T>
__global__ void __launch_bounds__(256) reduce_outer_kernel(const T* __restrict__ x, T* __restrict__ part, ReduceGeom g,
                                                           FastDiv dk0, FastDiv dr1, FastDiv dct, int vec_ok) {
    constexpr int V = VecOf<T>::N;
    __shared__ T red[8][32 * V + 1];
    const int cg = threadIdx.x & 31, rl = threadIdx.x >> 5;
    uint32_t o, ct;  // kept outer index kb*K0 + k0 and column tile, both folded into grid.x
    dct.divmod(blockIdx.x, o, ct);
    const int64_t col0 = ((int64_t)ct * 32 + cg) * V;
    const int p = blockIdx.y;
    uint32_t kb, k0;
    dk0.divmod(o, kb, k0);
    const uint32_t rows = (uint32_t)(g.R0 * g.R1);
    const uint32_t len = (rows + g.parts - 1) / g.parts;
    const uint32_t r_begin = (uint32_t)p * len;
    const uint32_t r_end = r_begin + len < rows ? r_begin + len : rows;
    const int64_t r0_stride = g.K0 * g.R1 * g.K1;
    const T* base = x + ((int64_t)kb * g.R0 * g.K0 + k0) * g.R1 * g.K1 + col0;
    T acc[4][V];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int e = 0; e < V; ++e) acc[u][e] = T(0);
    if (col0 < g.K1) {
        auto row_ptr = [&](uint32_t r) {
            uint32_t r0, r1;
            dr1.divmod(r, r0, r1);
            return base + (int64_t)r0 * r0_stride + (int64_t)r1 * g.K1;
        };
        uint32_t r = r_begin + rl;
        if (vec_ok) {
            for (; r + 24 < r_end; r += 32) {
                T v[4][V];
#pragma unroll
                for (int u = 0; u < 4; ++u) vload<T>(row_ptr(r + 8 * u), v[u]);
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int e = 0; e < V; ++e) acc[u][e] += v[u][e];
            }
            for (; r < r_end; r += 8) {
                T v[V];
                vload<T>(row_ptr(r), v);
#pragma unroll
                for (int e = 0; e < V; ++e) acc[0][e] += v[e];
            }
        } else {
            for (; r < r_end; r += 8) {
                const T* src = row_ptr(r);
#pragma unroll
                for (int e = 0; e < V; ++e)
                    if (col0 + e < g.K1) acc[0][e] += src[e];
            }
        }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) red[rl][cg * V + e] = (acc[0][e] + acc[1][e]) + (acc[2][e] + acc[3][e]);
    __syncthreads();
    if (rl == 0 && col0 < g.K1) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
            if (col0 + e < g.K1) {
                T s = T(0);
                for (int w = 0; w < 8; ++w) s += red[w][cg * V + e];
                part[(int64_t)p * g.outputs + (int64_t)o * g.K1 + col0 + e] = s;
            }
        }
    }
}

template <typename T>
__global__ void reduce_finish_kernel(const T* __restrict__ part, T* __restrict__ out, int64_t outputs, int parts) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < outputs; i += (int64_t)gridDim.x * blockDim.x) {
        T s = part[i];
        for (int p = 1; p < parts; ++p) s += part[(int64_t)p * outputs + i];
        out[i] = s;
    }
}

static int collapse_axes(Context* c, const int64_t* shape, int ndim, const int* axes, int naxes, ReduceGeom& g,
                         bool& any_reduced) {
    FXB_CHECK_ARG(c, ndim >= 0 && ndim <= 8 && (ndim == 0 || shape != nullptr), "sum_axes supports up to 8 dimensions");
    bool red[8] = {};
    for (int i = 0; i < naxes; ++i) {
        if (axes[i] < 0 || axes[i] >= ndim)
            return fail(c, FXB_ERR_INVALID_ARGUMENT,
                        "Axis " + std::to_string(axes[i]) + " is out of bounds for tensor with " + std::to_string(ndim) +
                            " dimensions");
        red[axes[i]] = true;
    }
    std::vector<std::pair<bool, int64_t>> groups;  // (reduced?, size), size-1 dims dropped, neighbours merged
    for (int i = 0; i < ndim; ++i) {
        FXB_CHECK_ARG(c, shape[i] >= 0, "negative dimension");
        if (shape[i] == 1) continue;
        if (!groups.empty() && groups.back().first == red[i]) groups.back().second *= shape[i];
        else groups.emplace_back(red[i], shape[i]);
    }
    // right-aligned placement into the slots [KB, R0, K0, R1, K1]
    int64_t slot[5] = {1, 1, 1, 1, 1};
    const bool slot_red[5] = {false, true, false, true, false};
    int s = 4;
    for (int gi = (int)groups.size() - 1; gi >= 0; --gi) {
        while (s >= 0 && slot_red[s] != groups[gi].first) --s;
        if (s < 0) return fail(c, FXB_ERR_UNSUPPORTED, "sum_axes: more than two separate runs of reduced axes");
        slot[s] = groups[gi].second;
        --s;
    }
    g.KB = slot[0]; g.R0 = slot[1]; g.K0 = slot[2]; g.R1 = slot[3]; g.K1 = slot[4];
    g.outputs = g.KB * g.K0 * g.K1;
    any_reduced = false;
    for (auto& gr : groups) any_reduced |= gr.first;
    return FXB_OK;
}

static int pick_parts(const Context* c, const ReduceGeom& g) {
    const int64_t per_out = g.R0 * g.R1;
    int64_t units = g.K1 > 1 ? g.KB * g.K0 * ((g.K1 + 127) / 128) : g.KB * g.K0;
    if (units <= 0) units = 1;
    // aim for >= 4 CTAs per SM (8 when the inner axis is reduced: those CTAs keep fewer bytes in flight),
    // but keep every part large enough to amortise its reduction
    const int64_t min_len = g.K1 > 1 ? 64 : 8192;
    int64_t parts = ((int64_t)c->sm_count * (g.K1 > 1 ? 4 : 8) + units - 1) / units;
    parts = std::min<int64_t>(parts, std::max<int64_t>(1, per_out / min_len));
    parts = std::max<int64_t>(1, std::min<int64_t>(parts, 1024));
    return (int)parts;
}

template <typename T>
static int sum_axes_impl(Context* c, const T* x, const int64_t* shape, int ndim, const int* axes, int naxes, T* out,
                         void* ws, size_t ws_bytes, cudaStream_t st) {
    ReduceGeom g;
    bool any = false;
    int rc = collapse_axes(c, shape, ndim, axes, naxes, g, any);
    if (rc) return rc;
    int64_t total = 1;
    for (int i = 0; i < ndim; ++i) total *= shape[i];
    if (g.outputs == 0) return FXB_OK;
    FXB_CHECK_ARG(c, out != nullptr && (total == 0 || x != nullptr), "sum_axes: null buffer");
    if (total == 0) {
        FXB_CUDA_OK(c, cudaMemsetAsync(out, 0, (size_t)g.outputs * sizeof(T), st));
        return FXB_OK;
    }
    if (!any) {  // nothing to reduce: a copy
        return launch_ew<T, 1>(c, x, (const T*)nullptr, out, total, ScaleF<T>{T(1)}, st, "sum_axes(copy)");
    }
    g.parts = pick_parts(c, g);
    const size_t need = g.parts > 1 ? (size_t)g.parts * g.outputs * sizeof(T) : 0;
    if (need > ws_bytes || (need > 0 && ws == nullptr)) {
        // fall back to fewer parts rather than failing: the result is the same, only slower
        g.parts = ws == nullptr ? 1 : (int)std::max<size_t>(1, ws_bytes / ((size_t)g.outputs * sizeof(T)));
    }
    T* part = g.parts > 1 ? static_cast<T*>(ws) : out;
    constexpr int V = VecOf<T>::N;
    const bool al = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    FXB_CHECK_ARG(c, g.R0 * g.R1 < ((int64_t)1 << 31), "sum_axes: more than 2^31-1 elements per output");
    if (g.K1 == 1) {
        FXB_CHECK_ARG(c, g.KB * g.K0 < ((int64_t)1 << 31), "sum_axes: too many outputs");
        const int vec_ok = al && (g.R1 % V == 0);
        dim3 grid((unsigned)(g.KB * g.K0), (unsigned)g.parts);
        reduce_inner_kernel<T><<<grid, 256, 0, st>>>(x, part, g, FastDiv((uint32_t)g.K0),
                                                     FastDiv((uint32_t)(vec_ok ? g.R1 / V : g.R1)), vec_ok);
    } else {
        const int vec_ok = al && (g.K1 % V == 0);
        const int64_t ctiles = (g.K1 + 32 * V - 1) / (32 * V);
        FXB_CHECK_ARG(c, ctiles * g.KB * g.K0 < ((int64_t)1 << 31), "sum_axes: too many outputs");
        dim3 grid((unsigned)(ctiles * g.KB * g.K0), (unsigned)g.parts);
        reduce_outer_kernel<T><<<grid, 256, 0, st>>>(x, part, g, FastDiv((uint32_t)g.K0), FastDiv((uint32_t)g.R1),
                                                     FastDiv((uint32_t)ctiles), vec_ok);
    }
    rc = launch_status(c, "reduce_sum stage 1");
    if (rc) return rc;
    if (g.parts > 1) {
        const int blocks = (int)std::min<int64_t>((g.outputs + 255) / 256, (int64_t)c->sm_count * 4);
        reduce_finish_kernel<T><<<blocks, 256, 0, st>>>(part, out, g.outputs, g.parts);
        rc = launch_status(c, "reduce_sum stage 2");
    }
    return rc;
}

static size_t sum_axes_ws_one(Context* c, const int64_t* shape, int ndim, const int* axes, int naxes, size_t elem) {
    ReduceGeom g;
    bool any = false;
    if (collapse_axes(c, shape, ndim, axes, naxes, g, any) != FXB_OK || !any || g.outputs == 0) return 0;
    g.parts = pick_parts(c, g);
    return g.parts > 1 ? (size_t)g.parts * g.outputs * elem : 0;
}

// One launch pair handles at most two separate runs of reduced axes.  With more (a 5-D or larger
// tensor reduced over alternating axes) the two innermost runs are reduced first into an
// intermediate tensor at the front of the workspace, and the rest in a second round.
// Returns false when the axes form at most two runs (or are invalid: the single-round code reports that).
struct AxisSplit {
    int first_axes[8], nfirst, rest_axes[8], nrest, mid_ndim;
    int64_t mid_shape[8], mid_elems;
};
static bool split_reduced_runs(const int64_t* shape, int ndim, const int* axes, int naxes, AxisSplit& sp) {
    if (ndim < 5 || ndim > 8) return false;
    bool red[8] = {};
    for (int i = 0; i < naxes; ++i) {
        if (axes[i] < 0 || axes[i] >= ndim) return false;
        red[axes[i]] = true;
    }
    int run_of[8], runs = 0;
    bool in_run = false;
    for (int i = 0; i < ndim; ++i) {
        run_of[i] = -1;
        if (shape[i] == 1) continue;  // size-1 dimensions neither join nor separate runs
        if (red[i]) {
            if (!in_run) { ++runs; in_run = true; }
            run_of[i] = runs - 1;
        } else {
            in_run = false;
        }
    }
    if (runs <= 2) return false;
    sp.nfirst = sp.nrest = sp.mid_ndim = 0;
    sp.mid_elems = 1;
    for (int i = 0; i < ndim; ++i) {
        const bool first = red[i] && (shape[i] == 1 || run_of[i] >= runs - 2);
        if (first) { sp.first_axes[sp.nfirst++] = i; continue; }
        if (red[i]) sp.rest_axes[sp.nrest++] = sp.mid_ndim;
        sp.mid_shape[sp.mid_ndim++] = shape[i];
        sp.mid_elems *= shape[i];
    }
    return true;
}
static size_t align_up256s(size_t v) { return (v + 255) & ~(size_t)255; }

static size_t sum_axes_ws(Context* c, const int64_t* shape, int ndim, const int* axes, int naxes, size_t elem) {
    AxisSplit sp;
    if (!split_reduced_runs(shape, ndim, axes, naxes, sp)) return sum_axes_ws_one(c, shape, ndim, axes, naxes, elem);
    const size_t a = sum_axes_ws_one(c, shape, ndim, sp.first_axes, sp.nfirst, elem);
    const size_t b = sum_axes_ws(c, sp.mid_shape, sp.mid_ndim, sp.rest_axes, sp.nrest, elem);
    return align_up256s((size_t)sp.mid_elems * elem) + std::max(a, b);
}

template <typename T>
static int sum_axes_any(Context* c, const T* x, const int64_t* shape, int ndim, const int* axes, int naxes, T* out,
                        void* ws, size_t ws_bytes, cudaStream_t st) {
    AxisSplit sp;
    if (shape == nullptr || axes == nullptr || !split_reduced_runs(shape, ndim, axes, naxes, sp))
        return sum_axes_impl<T>(c, x, shape, ndim, axes, naxes, out, ws, ws_bytes, st);
    if (sp.mid_elems == 0) return FXB_OK;
    const size_t mid_bytes = align_up256s((size_t)sp.mid_elems * sizeof(T));
    if (ws == nullptr || ws_bytes < mid_bytes)
        return fail(c, FXB_ERR_WORKSPACE,
                    "sum_axes: more than two separate runs of reduced axes need a workspace of fxb_sum_axes_workspace_bytes");
    T* mid = static_cast<T*>(ws);
    char* rest_ws = static_cast<char*>(ws) + mid_bytes;
    const size_t rest_bytes = ws_bytes - mid_bytes;
    const int rc = sum_axes_impl<T>(c, x, shape, ndim, sp.first_axes, sp.nfirst, mid, rest_ws, rest_bytes, st);
    if (rc) return rc;
    return sum_axes_any<T>(c, mid, sp.mid_shape, sp.mid_ndim, sp.rest_axes, sp.nrest, out, rest_ws, rest_bytes, st);
}

// ------------------------------------------------------------------------------------------
// Softmax cross-entropy, mean reduction, forward + gradient w.r.t. the logits in one launch.
// Each warp walks rows; every CTA leaves its loss sum in `partials`, the CTA that arrives last
// adds them in CTA order (deterministic) and writes the mean.
template <typename T> __device__ __forceinline__ T dev_log(T x);
template <> __device__ __forceinline__ float dev_log<float>(float x) { return logf(x); }
template <> __device__ __forceinline__ double dev_log<double>(double x) { return log(x); }
template <typename T> __device__ __forceinline__ T lowest_val();
template <> __device__ __forceinline__ float lowest_val<float>() { return -3.402823466e+38f; }
template <> __device__ __forceinline__ double lowest_val<double>() { return -1.7976931348623157e+308; }

constexpr int CE_MAX_BLOCKS = 960;  // per-CTA loss partials live in the handle's 8 KB scratch block

template <typename T>
__global__ void __launch_bounds__(256) softmax_ce_kernel(const T* __restrict__ logits, const T* __restrict__ targets,
                                                         T* __restrict__ loss_out, T* __restrict__ dlogits, int64_t B,
                                                         int64_t C, T grad_scale, T* __restrict__ partials,
                                                         unsigned int* __restrict__ counter) {
    __shared__ T wsum[8];
    __shared__ bool is_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T eps = T(1e-8), one_m = T(1.0 - 1e-8);
    const T inv_b = T(1.0 / (double)B);
    T loss_acc = T(0);
    for (int64_t row = (int64_t)blockIdx.x * 8 + warp; row < B; row += (int64_t)gridDim.x * 8) {
        const T* z = logits + row * C;
        const T* t = targets + row * C;
        T mx = lowest_val<T>();
        for (int64_t j = lane; j < C; j += 32) mx = z[j] > mx ? z[j] : mx;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { const T other = __shfl_xor_sync(0xffffffffu, mx, o); mx = other > mx ? other : mx; }
        T s = T(0);
        for (int64_t j = lane; j < C; j += 32) s += dev_exp<T>(z[j] - mx);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        T rowl = T(0), dot = T(0);
        for (int64_t j = lane; j < C; j += 32) {
            const T p = dev_exp<T>(z[j] - mx) / s;
            const T pc = p < eps ? eps : (p > one_m ? one_m : p);
            rowl += t[j] * dev_log<T>(pc);
            const T mask = (p >= eps ? T(1) : T(0)) * (p <= one_m ? T(1) : T(0));
            const T gj = ((-inv_b) * t[j]) / pc * mask;
            dot += gj * p;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            rowl += __shfl_xor_sync(0xffffffffu, rowl, o);
            dot += __shfl_xor_sync(0xffffffffu, dot, o);
        }
        loss_acc += -rowl;
        if (dlogits != nullptr) {
            for (int64_t j = lane; j < C; j += 32) {
                const T p = dev_exp<T>(z[j] - mx) / s;
                const T pc = p < eps ? eps : (p > one_m ? one_m : p);
                const T mask = (p >= eps ? T(1) : T(0)) * (p <= one_m ? T(1) : T(0));
                const T gj = ((-inv_b) * t[j]) / pc * mask;
                dlogits[row * C + j] = (p * (gj - dot)) * grad_scale;
            }
        }
    }
    if (lane == 0) wsum[warp] = loss_acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        T total = T(0);
        for (int w = 0; w < 8; ++w) total += wsum[w];
        partials[blockIdx.x] = total;
        __threadfence();
        const unsigned int done = atomicAdd(counter, 1u);
        is_last = done == gridDim.x - 1;
    }
    __syncthreads();
    if (is_last && threadIdx.x == 0) {
        __threadfence();
        T total = T(0);
        for (unsigned int b = 0; b < gridDim.x; ++b) total += reinterpret_cast<volatile T*>(partials)[b];
        *loss_out = total * inv_b;
        *counter = 0u;  // ready for the next launch on this handle
    }
}

// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) sgd_kernel(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ mom,
                                                  int64_t n, T lr, T momentum, T wd, int nesterov, T gscale) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        T gi = g[i];
        if (gscale != T(1)) gi *= gscale;
        const T pi = p[i];
        const T eg = wd == T(0) ? gi : gi + pi * wd;
        if (momentum != T(0)) {
            const T mi = mom[i] * momentum + eg;
            mom[i] = mi;
            const T upd = nesterov ? mi * momentum + eg : mi;
            p[i] = pi - upd * lr;
        } else {
            p[i] = pi - eg * lr;
        }
    }
}

template <typename T> __device__ __forceinline__ T dev_sqrt(T x);
template <> __device__ __forceinline__ float dev_sqrt<float>(float x) { return sqrtf(x); }
template <> __device__ __forceinline__ double dev_sqrt<double>(double x) { return sqrt(x); }

template <typename T>
__device__ __forceinline__ void adam_update(T& p, T g, T& m, T& v, T lr, T b1, T b2, T omb1, T omb2, T eps, T wd, T bc1, T bc2,
                                            T gscale) {
    if (gscale != T(1)) g *= gscale;
    const T mi = m * b1 + g * omb1;
    const T vi = v * b2 + (g * g) * omb2;
    m = mi;
    v = vi;
    const T den = dev_sqrt<T>(vi / bc2) + eps;
    const T upd = ((mi / bc1) / den) * lr;
    p = wd != T(0) ? (p - upd) - p * (wd * lr) : p - upd;
}
// One 16-byte vector of each array per thread step when the four arrays are 16-byte aligned, a scalar tail otherwise.
template <typename T>
__device__ __forceinline__ void adam_range(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ m, T* __restrict__ v,
                                           int64_t n, T lr, T b1, T b2, T eps, T wd, T bc1, T bc2, T gscale, int vec_ok) {
    constexpr int V = VecOf<T>::N;
    const T omb1 = T(1) - b1, omb2 = T(1) - b2;
    const int64_t tid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x, nth = (int64_t)gridDim.x * blockDim.x;
    int64_t done = 0;
    if (vec_ok) {
        const int64_t nvec = n / V;
        for (int64_t i = tid; i < nvec; i += nth) {
            T pv[V], gv[V], mv[V], vv[V];
            vload<T>(p + i * V, pv);
            vload<T>(g + i * V, gv);
            vload<T>(m + i * V, mv);
            vload<T>(v + i * V, vv);
#pragma unroll
            for (int e = 0; e < V; ++e) adam_update<T>(pv[e], gv[e], mv[e], vv[e], lr, b1, b2, omb1, omb2, eps, wd, bc1, bc2, gscale);
            vstore<T>(p + i * V, pv);
            vstore<T>(m + i * V, mv);
            vstore<T>(v + i * V, vv);
        }
        done = nvec * V;
    }
    for (int64_t i = done + tid; i < n; i += nth) adam_update<T>(p[i], g[i], m[i], v[i], lr, b1, b2, omb1, omb2, eps, wd, bc1, bc2, gscale);
}
template <typename T>
__global__ void __launch_bounds__(256) adam_kernel(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ m,
                                                   T* __restrict__ v, int64_t n, T lr, T b1, T b2, T eps, T wd, T bc1,
                                                   T bc2, T gscale, int vec_ok) {
    adam_range<T>(p, g, m, v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale, vec_ok);
}

// Adam with the step count in device memory, for a train step that is replayed from a CUDA graph
// (kernel arguments are frozen at capture time, the bias corrections 1 - beta^t change every step).
// *step_dev holds the number of steps done so far; the update uses t = *step_dev + 1.  The counter is
// advanced by the one-thread kernel launched right after (stream order keeps every block of the update
// on the old value).
template <typename T> __device__ __forceinline__ T dev_pow(T b, T e);
template <> __device__ __forceinline__ float dev_pow<float>(float b, float e) { return powf(b, e); }
template <> __device__ __forceinline__ double dev_pow<double>(double b, double e) { return pow(b, e); }

template <typename T>
__global__ void __launch_bounds__(256) adam_devcount_kernel(T* __restrict__ p, const T* __restrict__ g, T* __restrict__ m,
                                                            T* __restrict__ v, int64_t n, T lr, T b1, T b2, T eps, T wd,
                                                            const long long* __restrict__ step_dev, T gscale, int vec_ok) {
    const T t = (T)(*step_dev + 1);
    const T b1p = dev_pow<T>(b1, t), b2p = dev_pow<T>(b2, t);
    const T bc1 = T(1) - (b1p > T(1e-8) ? b1p : T(1e-8)), bc2 = T(1) - (b2p > T(1e-8) ? b2p : T(1e-8));
    adam_range<T>(p, g, m, v, n, lr, b1, b2, eps, wd, bc1, bc2, gscale, vec_ok);
}
__global__ void advance_step_kernel(long long* step_dev) { *step_dev += 1; }

static int aligned16_all(const void* a, const void* b, const void* c, const void* d) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
             reinterpret_cast<uintptr_t>(d)) & 15) == 0;
}
static int flat_grid(const Context* c, int64_t n) {
    return (int)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)c->sm_count * 8));
}

// ------------------------------------------------------------------------------------------
// Sum over axes for callers that cannot allocate.
//
// fxb_sum_axes_f32 keeps its stage-one partial sums in a workspace the caller takes from its
// memory pool.  Some callers of this library have no pool to ask at the moment they need a sum:
// code that runs while the pool's mutex is held (a Drop handler returning buffers, the pool's own
// eviction path), and an out-of-memory handler that still wants a loss or gradient-norm value for
// its report after the pool has refused a request.  Calling cudaMalloc there is not an option
// either (it synchronises the device and can fail for the same reason the pool did).
// For them the same two kernels run with their partial sums in the fixed array below, which is
// part of the library image: every GPU that loads the library holds these 512 KiB until exit.
constexpr size_t STATIC_SCRATCH_BYTES = (size_t)512 << 10;
static __device__ __align__(256) unsigned char g_sum_scratch[STATIC_SCRATCH_BYTES];

// `g_sum_scratch` in host code is only a host-side handle for the symbol, not a device address.
// fxb_create calls this once per handle, with the handle's device current, and keeps the device
// address in the context, so that the entry point below never touches the module loader or the
// current device (its callers may be inside an out-of-memory handler).
int resolve_static_scratch(Context* c) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_sum_scratch);
    if (e != cudaSuccess || p == nullptr)
        return fail(c, FXB_ERR_CUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
    c->static_scratch = p;
    return FXB_OK;
}

}  // namespace fxb

// Same result, bit for bit, as fxb_sum_axes_f32 with a workspace of fxb_sum_axes_workspace_bytes.
//  - Allocates nothing: no cudaMalloc / cudaFree / pool call, the partial sums live in the
//    library's static 512 KiB device array.
//  - A reduction whose partial sums need more than that is refused with FXB_ERR_WORKSPACE
//    (nothing is launched); use fxb_sum_axes_f32 with a pool workspace for those.
//  - The array's device address was looked up by fxb_create (cudaGetSymbolAddress with the handle's
//    device current), so this call touches neither the module loader nor the current device.
//  - Every call on a device shares the one array and leaves its partial sums behind.  Nothing
//    in it has to be zero beforehand (stage one overwrites every slot stage two reads), but two
//    calls that overlap on the GPU (different streams, no ordering) would race on it.
extern "C" int fxb_sum_axes_static_scratch_f32(fxb_handle_t h, const float* x, const int64_t* shape, int ndim,
                                               const int* axes, int naxes, float* out, fxb_stream_t stream) {
    if (h == nullptr) return fxb::fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle");
    fxb::Context* c = reinterpret_cast<fxb::Context*>(h);
    const size_t need = fxb::sum_axes_ws(c, shape, ndim, axes, naxes, sizeof(float));
    if (need > fxb::STATIC_SCRATCH_BYTES)
        return fxb::fail(c, FXB_ERR_WORKSPACE,
                         "fxb_sum_axes_static_scratch_f32: this reduction needs " + std::to_string(need) +
                             " bytes of partial sums, the static scratch holds " +
                             std::to_string(fxb::STATIC_SCRATCH_BYTES) + "; use fxb_sum_axes_f32 with a workspace");
    if (c->static_scratch == nullptr)
        return fxb::fail(c, FXB_ERR_CUDA, "fxb_sum_axes_static_scratch_f32: the static scratch address was not resolved by fxb_create");
    return fxb::sum_axes_any<float>(c, x, shape, ndim, axes, naxes, out, c->static_scratch, fxb::STATIC_SCRATCH_BYTES,
                                    static_cast<cudaStream_t>(stream));
}


using namespace fxb;
#define CTX(h) reinterpret_cast<fxb::Context*>(h)
#define ST(s) static_cast<cudaStream_t>(s)
#define NEED_HANDLE(h) \
    if ((h) == nullptr) return fxb::fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle")

#define FXB_STREAM_API(SUF, T)                                                                                          \
    extern "C" int fxb_act_fwd_##SUF(fxb_handle_t h, const T* x, T* y, int64_t n, int act, fxb_stream_t s) {            \
        NEED_HANDLE(h);                                                                                                 \
        FXB_CHECK_ARG(CTX(h), act >= FXB_ACT_NONE && act <= FXB_ACT_TANH, "Unknown activation code");                   \
        return launch_ew<T, 1>(CTX(h), x, (const T*)nullptr, y, n, ActFwdF<T>{act}, ST(s), "activation forward");       \
    }                                                                                                                   \
    extern "C" int fxb_act_bwd_##SUF(fxb_handle_t h, const T* dy, const T* aux, T* dx, int64_t n, int act,              \
                                     fxb_stream_t s) {                                                                  \
        NEED_HANDLE(h);                                                                                                 \
        FXB_CHECK_ARG(CTX(h), act >= FXB_ACT_NONE && act <= FXB_ACT_TANH, "Unknown activation code");                   \
        return launch_ew<T, 2>(CTX(h), dy, aux, dx, n, ActBwdF<T>{act, CTX(h)->sigmoid_grad_math}, ST(s),               \
                               "activation backward");                                                                  \
    }                                                                                                                   \
    extern "C" int fxb_add_##SUF(fxb_handle_t h, const T* a, const T* b, T* out, int64_t n, fxb_stream_t s) {           \
        NEED_HANDLE(h);                                                                                                 \
        return launch_ew<T, 2>(CTX(h), a, b, out, n, AddF<T>{}, ST(s), "add");                                          \
    }                                                                                                                   \
    extern "C" int fxb_mul_##SUF(fxb_handle_t h, const T* a, const T* b, T* out, int64_t n, fxb_stream_t s) {           \
        NEED_HANDLE(h);                                                                                                 \
        return launch_ew<T, 2>(CTX(h), a, b, out, n, MulF<T>{}, ST(s), "mul");                                          \
    }                                                                                                                   \
    extern "C" int fxb_axpby_##SUF(fxb_handle_t h, T alpha, const T* x, T beta, const T* y, T* out, int64_t n,          \
                                   fxb_stream_t s) {                                                                    \
        NEED_HANDLE(h);                                                                                                 \
        if (y == nullptr || beta == T(0))                                                                               \
            return launch_ew<T, 1>(CTX(h), x, (const T*)nullptr, out, n, ScaleF<T>{alpha}, ST(s), "axpby");             \
        return launch_ew<T, 2>(CTX(h), x, y, out, n, AxpbyF<T>{alpha, beta}, ST(s), "axpby");                           \
    }                                                                                                                   \
    extern "C" int fxb_greater_scalar_##SUF(fxb_handle_t h, const T* x, T sc, T* out, int64_t n, fxb_stream_t s) {      \
        NEED_HANDLE(h);                                                                                                 \
        return launch_ew<T, 1>(CTX(h), x, (const T*)nullptr, out, n, GreaterF<T>{sc}, ST(s), "greater_scalar");         \
    }                                                                                                                   \
    extern "C" int fxb_bias_add_##SUF(fxb_handle_t h, T* y, const T* bias, int64_t outer, int64_t channels,             \
                                      int64_t plane, fxb_stream_t s) {                                                  \
        NEED_HANDLE(h);                                                                                                 \
        FXB_CHECK_ARG(CTX(h), outer >= 0 && channels > 0 && plane > 0, "bias_add: bad shape");                          \
        const int64_t n = outer * channels * plane;                                                                     \
        FXB_CHECK_ARG(CTX(h), n < ((int64_t)1 << 31), "bias_add: tensor has more than 2^31-1 elements");                \
        if (n == 0) return FXB_OK;                                                                                      \
        FXB_CHECK_ARG(CTX(h), y && bias, "bias_add: null buffer");                                                      \
        bias_add_kernel<T><<<flat_grid(CTX(h), n), EW_THREADS, 0, ST(s)>>>(y, bias, n, FastDiv((uint32_t)plane),        \
                                                                          (int)channels);                               \
        return launch_status(CTX(h), "bias_add");                                                                       \
    }                                                                                                                   \
    extern "C" int fxb_sum_axes_##SUF(fxb_handle_t h, const T* x, const int64_t* shape, int ndim, const int* axes,      \
                                      int naxes, T* out, void* ws, size_t wsb, fxb_stream_t s) {                        \
        NEED_HANDLE(h);                                                                                                 \
        return sum_axes_any<T>(CTX(h), x, shape, ndim, axes, naxes, out, ws, wsb, ST(s));                               \
    }                                                                                                                   \
    extern "C" int fxb_sum_all_##SUF(fxb_handle_t h, const T* x, int64_t n, T* out, void* ws, size_t wsb,               \
                                     fxb_stream_t s) {                                                                  \
        NEED_HANDLE(h);                                                                                                 \
        const int64_t shape[1] = {n};                                                                                   \
        const int axes[1] = {0};                                                                                        \
        return sum_axes_impl<T>(CTX(h), x, shape, 1, axes, 1, out, ws, wsb, ST(s));                                     \
    }                                                                                                                   \
    extern "C" int fxb_softmax_ce_##SUF(fxb_handle_t h, const T* logits, const T* targets, T* loss_out, T* dlogits,     \
                                        int64_t B, int64_t C, T grad_scale, fxb_stream_t s) {                           \
        NEED_HANDLE(h);                                                                                                 \
        FXB_CHECK_ARG(CTX(h), B > 0 && C > 0, "softmax_ce: batch and class counts must be positive");                   \
        FXB_CHECK_ARG(CTX(h), logits && targets && loss_out, "softmax_ce: null buffer");                                \
        const int ce_blocks = (int)std::min<int64_t>((B + 7) / 8, std::min<int>(CE_MAX_BLOCKS, CTX(h)->sm_count * 4));   \
        T* ce_part = reinterpret_cast<T*>(static_cast<char*>(CTX(h)->d_scratch) + 64);                                  \
        unsigned int* ce_cnt = reinterpret_cast<unsigned int*>(CTX(h)->d_scratch);                                      \
        softmax_ce_kernel<T><<<ce_blocks, 256, 0, ST(s)>>>(logits, targets, loss_out, dlogits, B, C, grad_scale,        \
                                                          ce_part, ce_cnt);                                             \
        return launch_status(CTX(h), "softmax_ce");                                                                     \
    }                                                                                                                   \
    extern "C" int fxb_sgd_step_##SUF(fxb_handle_t h, T* p, const T* g, T* mom, int64_t n, T lr, T momentum, T wd,      \
                                      int nesterov, T gscale, fxb_stream_t s) {                                         \
        NEED_HANDLE(h);                                                                                                 \
        if (n == 0) return FXB_OK;                                                                                      \
        FXB_CHECK_ARG(CTX(h), n > 0 && p && g && (momentum == T(0) || mom), "sgd_step: bad arguments");                 \
        sgd_kernel<T><<<flat_grid(CTX(h), n), 256, 0, ST(s)>>>(p, g, mom, n, lr, momentum, wd, nesterov, gscale);       \
        return launch_status(CTX(h), "sgd_step");                                                                       \
    }                                                                                                                   \
    extern "C" int fxb_adam_step_##SUF(fxb_handle_t h, T* p, const T* g, T* m, T* v, int64_t n, T lr, T b1, T b2,       \
                                       T eps, T wd, int64_t step, T gscale, fxb_stream_t s) {                           \
        NEED_HANDLE(h);                                                                                                 \
        if (n == 0) return FXB_OK;                                                                                      \
        FXB_CHECK_ARG(CTX(h), n > 0 && p && g && m && v && step >= 1, "adam_step: bad arguments");                      \
        const T b1p = std::max((T)std::pow(b1, (T)step), (T)1e-8);                                                      \
        const T b2p = std::max((T)std::pow(b2, (T)step), (T)1e-8);                                                      \
        adam_kernel<T><<<flat_grid(CTX(h), n), 256, 0, ST(s)>>>(p, g, m, v, n, lr, b1, b2, eps, wd, T(1) - b1p,         \
                                                               T(1) - b2p, gscale, aligned16_all(p, g, m, v));          \
        return launch_status(CTX(h), "adam_step");                                                                      \
    }                                                                                                                   \
    extern "C" int fxb_adam_step_devcount_##SUF(fxb_handle_t h, T* p, const T* g, T* m, T* v, int64_t n, T lr, T b1,    \
                                                T b2, T eps, T wd, int64_t* step_dev, T gscale, fxb_stream_t s) {       \
        NEED_HANDLE(h);                                                                                                 \
        FXB_CHECK_ARG(CTX(h), n >= 0 && step_dev != nullptr && (n == 0 || (p && g && m && v)),                          \
                      "adam_step_devcount: bad arguments");                                                             \
        if (n > 0)                                                                                                      \
            adam_devcount_kernel<T><<<flat_grid(CTX(h), n), 256, 0, ST(s)>>>(                                           \
                p, g, m, v, n, lr, b1, b2, eps, wd, reinterpret_cast<const long long*>(step_dev), gscale,               \
                aligned16_all(p, g, m, v));                                                                             \
        advance_step_kernel<<<1, 1, 0, ST(s)>>>(reinterpret_cast<long long*>(step_dev));                                \
        return launch_status(CTX(h), "adam_step_devcount", n > 0 ? 2 : 1);                                              \
    }

FXB_STREAM_API(f32, float)
FXB_STREAM_API(f64, double)

extern "C" size_t fxb_sum_axes_workspace_bytes(fxb_handle_t h, const int64_t* shape, int ndim, const int* axes,
                                               int naxes, size_t elem) {
    if (!h) return 0;
    return sum_axes_ws(CTX(h), shape, ndim, axes, naxes, elem);
}
