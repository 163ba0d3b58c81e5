// Layout kernels of the C ABI: materialising a strided / broadcast view into contiguous memory,
// and the two ops built on it (transpose with an axis permutation, broadcast_to).
//
// The shape and stride arrays travel in the kernel parameters (no device copies of them), sizes are
// collapsed on the host (unit dimensions dropped, dimensions that are contiguous with respect to
// each other merged), and one of three kernels runs:
//   rows      the innermost output dimension is contiguous in the view too: 128-bit row copies;
//   transpose the innermost output dimension is strided in the view while another dimension has
//             stride 1 (any permutation that moves the innermost axis): 32 x 32 tiles through shared
//             memory, coalesced on both sides;
//   gather    everything else (e.g. a broadcast innermost dimension): one element per thread, the
//             reads of a warp fall on one or a few addresses.
// All three are pure data movement: results are bit-exact.
#include "fxb_common.cuh"

#include <algorithm>

namespace fxb {

constexpr int LAYOUT_MAX_DIMS = 8;

struct ViewGeom {
    int nd;                          // collapsed dimensions, outermost first
    FastDiv dshape[LAYOUT_MAX_DIMS]; // divisors by the output extents
    int64_t istride[LAYOUT_MAX_DIMS];  // view strides in elements (0 = broadcast)
    int64_t ostride[LAYOUT_MAX_DIMS];  // contiguous output strides
    int64_t total;
};

// Flattened index over dimensions [0, upto) (row-major) -> offsets in the view and in the output.
__device__ __forceinline__ void outer_offsets(const ViewGeom& g, uint32_t idx, int upto, int skip, int64_t& in_off,
                                              int64_t& out_off) {
    in_off = 0;
    out_off = 0;
#pragma unroll
    for (int d = LAYOUT_MAX_DIMS - 1; d >= 0; --d) {
        if (d >= upto || d == skip) continue;
        uint32_t q, r;
        g.dshape[d].divmod(idx, q, r);
        in_off += (int64_t)r * g.istride[d];
        out_off += (int64_t)r * g.ostride[d];
        idx = q;
    }
}

// rows: out[o][i] = in[off(o) + i]; one thread per vector of V elements of the innermost dimension.
template <typename T, int V>
__global__ void __launch_bounds__(256) materialize_rows_kernel(const T* __restrict__ in, T* __restrict__ out, ViewGeom g,
                                                               FastDiv dvecs, int inner) {
    const int64_t nvec = g.total / V;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < nvec; idx += (int64_t)gridDim.x * blockDim.x) {
        uint32_t o, iv;
        dvecs.divmod((uint32_t)idx, o, iv);
        int64_t in_off, out_off;
        outer_offsets(g, o, g.nd - 1, -1, in_off, out_off);
        const T* src = in + in_off + (int64_t)iv * V;
        T* dst = out + (int64_t)o * inner + (int64_t)iv * V;
        if (V == 1) {
            *dst = __ldg(src);
        } else {
            *reinterpret_cast<uint4*>(dst) = __ldg(reinterpret_cast<const uint4*>(src));
        }
    }
}

// transpose: dimension `jd` has stride 1 in the view, the innermost output dimension has stride `sl`.
// Block (32, 8) moves one 32 x 32 tile: read with threadIdx.x along jd, write with threadIdx.x along
// the innermost dimension.
template <typename T>
__global__ void __launch_bounds__(256) materialize_transpose_kernel(const T* __restrict__ in, T* __restrict__ out, ViewGeom g,
                                                                    int jd, int J, int L, FastDiv dtj, FastDiv dtl) {
    __shared__ T tile[32][33];
    __shared__ int64_t offs[2];
    uint32_t rest, tl, o, tj;
    dtl.divmod(blockIdx.x, rest, tl);
    dtj.divmod(rest, o, tj);
    if (threadIdx.x == 0 && threadIdx.y == 0) {  // the outer coordinates are the same for the whole tile
        int64_t io, oo;
        outer_offsets(g, o, g.nd - 1, jd, io, oo);
        offs[0] = io;
        offs[1] = oo;
    }
    __syncthreads();
    const int64_t in_off = offs[0], out_off = offs[1];
    const int64_t sl = g.istride[g.nd - 1], sjo = g.ostride[jd];
    const int j0 = (int)tj * 32, l0 = (int)tl * 32;
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        const int l = l0 + threadIdx.y + k, j = j0 + threadIdx.x;
        if (l < L && j < J) tile[threadIdx.y + k][threadIdx.x] = __ldg(in + in_off + j + (int64_t)l * sl);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 32; k += 8) {
        const int j = j0 + threadIdx.y + k, l = l0 + threadIdx.x;
        if (l < L && j < J) out[out_off + (int64_t)j * sjo + l] = tile[threadIdx.x][threadIdx.y + k];
    }
}

template <typename T>
__global__ void __launch_bounds__(256) materialize_gather_kernel(const T* __restrict__ in, T* __restrict__ out, ViewGeom g) {
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < g.total; idx += (int64_t)gridDim.x * blockDim.x) {
        int64_t in_off, out_off;
        outer_offsets(g, (uint32_t)idx, g.nd, -1, in_off, out_off);
        out[idx] = __ldg(in + in_off);
    }
}

template <typename T>
static int materialize_impl(Context* c, const T* in, T* out, const int64_t* shape, const int64_t* strides, int ndim,
                            cudaStream_t st) {
    FXB_CHECK_ARG(c, ndim >= 0 && ndim <= LAYOUT_MAX_DIMS, "materialize supports up to 8 dimensions");
    FXB_CHECK_ARG(c, ndim == 0 || (shape != nullptr && strides != nullptr), "materialize: null shape or strides");
    int64_t total = 1;
    for (int i = 0; i < ndim; ++i) {
        FXB_CHECK_ARG(c, shape[i] >= 0 && strides[i] >= 0, "materialize: negative extent or stride");
        total *= shape[i];
    }
    if (total == 0) return FXB_OK;
    FXB_CHECK_ARG(c, in != nullptr && out != nullptr, "materialize: null buffer");
    if (total >= ((int64_t)1 << 31)) return fail(c, FXB_ERR_UNSUPPORTED, "materialize: tensor has more than 2^31-1 elements");
    // collapse: drop unit dimensions, merge neighbours that are contiguous with respect to each other
    int64_t sh[LAYOUT_MAX_DIMS], sd[LAYOUT_MAX_DIMS];
    int nd = 0;
    for (int i = 0; i < ndim; ++i) {
        if (shape[i] == 1) continue;
        if (nd > 0 && sd[nd - 1] == strides[i] * shape[i]) {
            sh[nd - 1] *= shape[i];
            sd[nd - 1] = strides[i];
        } else {
            sh[nd] = shape[i];
            sd[nd] = strides[i];
            ++nd;
        }
    }
    if (nd == 0) { sh[0] = 1; sd[0] = 1; nd = 1; }
    ViewGeom g;
    g.nd = nd;
    g.total = total;
    int64_t os = 1;
    for (int d = LAYOUT_MAX_DIMS - 1; d >= 0; --d) {
        if (d < nd) {
            g.dshape[d].init((uint32_t)sh[d]);
            g.istride[d] = sd[d];
            g.ostride[d] = os;
            os *= sh[d];
        } else {
            g.dshape[d].init(1);
            g.istride[d] = 0;
            g.ostride[d] = 0;
        }
    }
    const int64_t inner = sh[nd - 1], sl = sd[nd - 1];
    auto blocks_for = [&](int64_t n) { return (int)std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, (int64_t)c->sm_count * 16)); };
    if (sl == 1 || inner == 1) {
        constexpr int V = 16 / (int)sizeof(T);
        bool vec = inner % V == 0 && (reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        for (int d = 0; d + 1 < nd; ++d) vec = vec && (sd[d] % V == 0);
        if (vec) {
            materialize_rows_kernel<T, V><<<blocks_for(total / V), 256, 0, st>>>(in, out, g, FastDiv((uint32_t)(inner / V)), (int)inner);
        } else {
            materialize_rows_kernel<T, 1><<<blocks_for(total), 256, 0, st>>>(in, out, g, FastDiv((uint32_t)inner), (int)inner);
        }
        return launch_status(c, "materialize_rows_kernel");
    }
    int jd = -1;
    for (int d = nd - 2; d >= 0; --d)
        if (sd[d] == 1 && sh[d] >= 8) { jd = d; break; }
    if (jd >= 0 && sl > 1) {
        const int64_t J = sh[jd], L = inner;
        const int64_t tj = (J + 31) / 32, tl = (L + 31) / 32;
        const int64_t outer = total / (J * L);
        const int64_t tiles = tj * tl * outer;
        if (tiles < ((int64_t)1 << 31)) {
            // the outer index enumerates every dimension but jd and the innermost one: jd's divisor must not split it
            ViewGeom gt = g;
            materialize_transpose_kernel<T><<<(unsigned)tiles, dim3(32, 8), 0, st>>>(in, out, gt, jd, (int)J, (int)L,
                                                                                      FastDiv((uint32_t)tj), FastDiv((uint32_t)tl));
            return launch_status(c, "materialize_transpose_kernel");
        }
    }
    materialize_gather_kernel<T><<<blocks_for(total), 256, 0, st>>>(in, out, g);
    return launch_status(c, "materialize_gather_kernel");
}

template <typename T>
static int transpose_impl(Context* c, const T* in, T* out, const int64_t* shape, int ndim, const int* axes, cudaStream_t st) {
    FXB_CHECK_ARG(c, ndim >= 0 && ndim <= LAYOUT_MAX_DIMS && (ndim == 0 || shape != nullptr), "transpose supports up to 8 dimensions");
    int64_t cs[LAYOUT_MAX_DIMS], oshape[LAYOUT_MAX_DIMS], ostr[LAYOUT_MAX_DIMS];
    int64_t s = 1;
    for (int i = ndim - 1; i >= 0; --i) { cs[i] = s; s *= shape[i]; }
    bool seen[LAYOUT_MAX_DIMS] = {};
    for (int i = 0; i < ndim; ++i) {
        const int a = axes ? axes[i] : ndim - 1 - i;  // no axes: reverse all (the 2-D matrix transpose)
        if (a < 0 || a >= ndim || seen[a])
            return fail(c, FXB_ERR_INVALID_ARGUMENT, "transpose: axes must be a permutation of 0.." + std::to_string(ndim - 1));
        seen[a] = true;
        oshape[i] = shape[a];
        ostr[i] = cs[a];
    }
    return materialize_impl<T>(c, in, out, oshape, ostr, ndim, st);
}

template <typename T>
static int broadcast_impl(Context* c, const T* in, const int64_t* in_shape, int in_ndim, T* out, const int64_t* out_shape,
                          int out_ndim, cudaStream_t st) {
    FXB_CHECK_ARG(c, in_ndim >= 0 && out_ndim <= LAYOUT_MAX_DIMS && in_ndim <= out_ndim, "broadcast_to: the target must have at least as many dimensions (up to 8)");
    FXB_CHECK_ARG(c, (in_ndim == 0 || in_shape) && (out_ndim == 0 || out_shape), "broadcast_to: null shape");
    int64_t str[LAYOUT_MAX_DIMS];
    int64_t s = 1;
    const int lead = out_ndim - in_ndim;
    for (int i = out_ndim - 1; i >= 0; --i) {
        if (i < lead) { str[i] = 0; continue; }
        const int64_t e = in_shape[i - lead];
        if (e == out_shape[i]) { str[i] = s; }
        else if (e == 1) { str[i] = 0; }
        else
            return fail(c, FXB_ERR_INVALID_ARGUMENT, "Cannot broadcast dimension of size " + std::to_string(e) + " to size " + std::to_string(out_shape[i]));
        s *= e;
    }
    return materialize_impl<T>(c, in, out, out_shape, str, out_ndim, st);
}

}  // namespace fxb

using namespace fxb;
#define CTX(h) reinterpret_cast<fxb::Context*>(h)
#define ST(s) static_cast<cudaStream_t>(s)
#define NEED_HANDLE(h) \
    if ((h) == nullptr) return fxb::fail(nullptr, FXB_ERR_INVALID_ARGUMENT, "null ferrox_b200 handle")

#define FXB_LAYOUT_API(SUF, T)                                                                                          \
    extern "C" int fxb_materialize_##SUF(fxb_handle_t h, const T* in, T* out, const int64_t* shape,                     \
                                         const int64_t* strides, int ndim, fxb_stream_t s) {                            \
        NEED_HANDLE(h);                                                                                                 \
        return materialize_impl<T>(CTX(h), in, out, shape, strides, ndim, ST(s));                                       \
    }                                                                                                                   \
    extern "C" int fxb_transpose_##SUF(fxb_handle_t h, const T* in, T* out, const int64_t* shape, int ndim,             \
                                       const int* axes, fxb_stream_t s) {                                               \
        NEED_HANDLE(h);                                                                                                 \
        return transpose_impl<T>(CTX(h), in, out, shape, ndim, axes, ST(s));                                            \
    }                                                                                                                   \
    extern "C" int fxb_broadcast_to_##SUF(fxb_handle_t h, const T* in, const int64_t* in_shape, int in_ndim, T* out,    \
                                          const int64_t* out_shape, int out_ndim, fxb_stream_t s) {                     \
        NEED_HANDLE(h);                                                                                                 \
        return broadcast_impl<T>(CTX(h), in, in_shape, in_ndim, out, out_shape, out_ndim, ST(s));                       \
    }

FXB_LAYOUT_API(f32, float)
FXB_LAYOUT_API(f64, double)
