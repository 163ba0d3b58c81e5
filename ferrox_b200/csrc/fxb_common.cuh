// Shared definitions of the ferrox_b200 CUDA library: status codes, the per-device context,
// host helpers, and the inline-PTX wrappers (mbarrier, tcgen05, TMEM) used by the kernels.
// Everything here targets sm_100a only.
#pragma once
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <string>

#include "../../include/ferrox_b200.h"

namespace fxb {

// ------------------------------------------------------------------------------------------
// Context: one per device, owned by the caller through fxb_create/fxb_destroy.  It holds no
// tensor memory; only a 64-byte device status block that kernels use to report a bounded
// wait that ran out (never a trap), and the configuration switches.
struct DeviceStatus {
    int code;        // 0 = ok, else FXB_ERR_DEVICE_TIMEOUT
    int where;       // which wait gave up (kernel-specific tag)
    int block_x, block_y, block_z;
    int pad[11];
};

struct Context {
    int device = 0;
    int sm_count = 148;
    int math_mode = FXB_MATH_3XTF32;
    int sigmoid_grad_math = 0;  // 0 = the reference's literal s*(s-1); 1 = s*(1-s)
    int operand_path = 0;       // FXB_PATH_*: which operand paths the f32 convolutions may take
    int drain_group = 4;        // 32-deep K stages accumulated in TMEM between two drains (fxb_set_accumulate_stages)
    DeviceStatus* d_status = nullptr;
    // 8 KB of handle-owned device scratch right after the status block (per-CTA partial sums of the
    // loss kernel + its arrival counter); used by one stream at a time, like the handle itself.
    void* d_scratch = nullptr;
    // device address of the library's static 512 KiB scratch array (fxb_sum_axes_static_scratch_f32),
    // resolved once by fxb_create with this device current
    void* static_scratch = nullptr;
    unsigned long long launches = 0;  // kernels launched through this handle
    std::string last_error;
};

extern thread_local std::string g_tls_error;  // defined in fxb_api.cu
int resolve_static_scratch(Context* c);        // defined in fxb_stream.cu, beside the array

inline int fail(Context* ctx, int code, const std::string& msg) {
    if (ctx) ctx->last_error = msg;
    g_tls_error = msg;
    return code;
}

#define FXB_CHECK_ARG(ctx, cond, msg)                                        \
    do {                                                                     \
        if (!(cond)) return ::fxb::fail((ctx), FXB_ERR_INVALID_ARGUMENT, (msg)); \
    } while (0)

#define FXB_CUDA_OK(ctx, expr)                                                                   \
    do {                                                                                         \
        cudaError_t e__ = (expr);                                                                \
        if (e__ != cudaSuccess)                                                                  \
            return ::fxb::fail((ctx), FXB_ERR_CUDA,                                              \
                               std::string(#expr) + ": " + cudaGetErrorString(e__));             \
    } while (0)

inline int launch_status(Context* ctx, const char* what, int kernels = 1) {
    if (ctx) ctx->launches += (unsigned long long)kernels;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(ctx, FXB_ERR_LAUNCH_FAILED, std::string("Kernel launch failed: ") + what + ": " + cudaGetErrorString(e));
    return FXB_OK;
}

// ------------------------------------------------------------------------------------------
// Exact unsigned division by a runtime constant: q = (n * mul) >> sh for 0 <= n < 2^31.
struct FastDiv {
    uint32_t d = 1, mul = 0, sh = 0;
    FastDiv() = default;
    explicit FastDiv(uint32_t div) { init(div); }
    void init(uint32_t div) {
        d = div ? div : 1;
        uint32_t l = 0;
        while ((1ull << l) < d) ++l;
        sh = 31 + l;
        mul = (uint32_t)(((1ull << sh) + d - 1) / d);
    }
    __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
        return (uint32_t)(((uint64_t)n * mul) >> sh);
    }
    __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
        q = div(n);
        r = n - q * d;
    }
};

// ------------------------------------------------------------------------------------------
// Activation helpers shared by epilogues, prologues and the streaming kernels.
// Codes match include/ferrox_b200.h (FXB_ACT_*).
template <typename T> __device__ __forceinline__ T dev_exp(T x);
template <> __device__ __forceinline__ float dev_exp<float>(float x) { return expf(x); }
template <> __device__ __forceinline__ double dev_exp<double>(double x) { return exp(x); }

template <typename T>
__device__ __forceinline__ T act_apply_full(T x, int act) {
    switch (act) {
        case FXB_ACT_RELU: return x > T(0) ? x : T(0);
        case FXB_ACT_SIGMOID: return T(1) / (T(1) + dev_exp<T>(-x));
        case FXB_ACT_TANH: {
            // Same branch structure as the reference CPU path (saturate beyond |x| > 20,
            // exp(-2x) form for x >= 0 and exp(2x) form for x < 0).
            if (x > T(20)) return T(1);
            if (x < T(-20)) return T(-1);
            if (x >= T(0)) { const T e = dev_exp<T>(-x * T(2)); return (T(1) - e) / (T(1) + e); }
            const T e = dev_exp<T>(x * T(2));
            return (e - T(1)) / (e + T(1));
        }
        default: return x;
    }
}

// The same function for the fused epilogues of the contraction kernels.  Those evaluate it once per
// accumulator register in fully unrolled code; with the exponentials inlined a single kernel grew to
// 200-350 KB of instructions and every tile's epilogue streamed its code from L2 (instruction-fetch
// stalls dominated).  Identity and ReLU stay inline, sigmoid and tanh go through one out-of-line copy.
template <typename T>
__device__ __noinline__ T act_apply_outlined(T x, int act) { return act_apply_full<T>(x, act); }
template <typename T>
__device__ __forceinline__ T act_apply(T x, int act) {
    if (act == FXB_ACT_NONE) return x;
    if (act == FXB_ACT_RELU) return x > T(0) ? x : T(0);
    return act_apply_outlined<T>(x, act);
}

// Factor multiplied into the upstream gradient.  `a` is the op input for relu and the op
// output for sigmoid / tanh.  sig_math = 0 reproduces the reference's s*(s-1).
template <typename T>
__device__ __forceinline__ T act_grad_factor(T a, int act, int sig_math) {
    switch (act) {
        case FXB_ACT_RELU: return a > T(0) ? T(1) : T(0);
        case FXB_ACT_SIGMOID: return sig_math ? a * (T(1) - a) : a * (a - T(1));
        case FXB_ACT_TANH: return -(a * a - T(1));
        default: return T(1);
    }
}

// ------------------------------------------------------------------------------------------
// PTX wrappers.
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// One attempt; the thread may be suspended by the hardware for up to `hint_ns` and is resumed as
// soon as the phase completes, so waiting warps do not compete for issue slots.
// (measured with 0, 200 and 4000 ns: no difference in any kernel)
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns = 4000u) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok;
}

// Bounded wait: spins on the barrier phase until it completes, another thread of the CTA has
// flagged an abort, or about `limit_cycles` SM cycles have passed.  On expiry it records the
// wait's tag in the device status block and raises the CTA-wide abort flag so every other
// role leaves its loop as well.  Returns false when the wait did not complete.
static __device__ __noinline__ bool mbar_wait_bounded_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  DeviceStatus* status, int tag, long long limit_cycles) {
    const long long t0 = clock64();
    int spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 63) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                if (atomicCAS(&status->code, 0, FXB_ERR_DEVICE_TIMEOUT) == 0) {
                    status->where = tag;
                    status->block_x = blockIdx.x;
                    status->block_y = blockIdx.y;
                    status->block_z = blockIdx.z;
                }
                return false;
            }
        }
    }
}
// The first attempt is inline; the spinning path is one out-of-line copy per kernel (the wait is
// used at a dozen places and its bookkeeping would otherwise be replicated at each of them).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  DeviceStatus* status, int tag,
                                                  long long limit_cycles = 4000000000LL) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_bounded_slow(bar, parity, abort_flag, status, tag, limit_cycles);
}

// 16-byte asynchronous global -> shared copy; `valid == false` writes 16 zero bytes instead.
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gsrc, bool valid) {
    const uint32_t nbytes = valid ? 16u : 0u;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(nbytes) : "memory");
}
// The same through L2 only (streaming data), and the thread-local group bookkeeping.
__device__ __forceinline__ void cp_async16_cg(uint32_t smem_dst, const void* gsrc, bool valid) {
    const uint32_t nbytes = valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(nbytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// Arrives on the mbarrier once every cp.async issued so far by this thread has landed; the arrival
// counts against the barrier's expected count.
__device__ __forceinline__ void cp_async_mbar_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Whole-warp instructions (.sync.aligned): call with all 32 lanes converged.
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc], TF32 inputs, FP32 accumulate.  One thread issues.
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Arrives on the mbarrier once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns; lane i of the warp receives TMEM lane (base+i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cvt_tf32_rna(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
// Four values -> their TF32 "hi" parts (round to nearest) and the exact remainders "lo", 16 bytes each.
__device__ __forceinline__ void store_split4(float* hi, float* lo, int64_t o, float v0, float v1, float v2, float v3) {
    uint4 h;
    h.x = cvt_tf32_rna(v0); h.y = cvt_tf32_rna(v1); h.z = cvt_tf32_rna(v2); h.w = cvt_tf32_rna(v3);
    *reinterpret_cast<uint4*>(hi + o) = h;
    *reinterpret_cast<float4*>(lo + o) = make_float4(v0 - __uint_as_float(h.x), v1 - __uint_as_float(h.y),
                                                     v2 - __uint_as_float(h.z), v3 - __uint_as_float(h.w));
}

// Where a forward kernel also leaves its output as the class slabs S[plane][n][iy][ix][4] (hi and lo) that the
// next convolution's tensor-map kernel reads (see split_image_to_class_slabs_kernel for the layout): geometry
// of that next layer's input.  hi == nullptr: nothing is emitted.  Only cells of real pixels are written; the
// padding cells of the buffer must have been zeroed once.
struct SlabEmit {
    float* hi = nullptr;
    float* lo = nullptr;
    int Q = 0, sw = 1, ph = 0, pw = 0, Wc = 0;
    FastDiv dsh, dsw;
    int64_t plane_stride = 0;  // floats between planes: N * Hc * Wc * 4
    int64_t img_stride = 0;    // floats between images of one plane: Hc * Wc * 4
};
// Offset (floats) of chunk 0 of pixel (y, x) of image n; chunk q (channels 4q..4q+3) lies q * plane_stride further.
__device__ __forceinline__ int64_t slab_cell_offset(const SlabEmit& e, int n, int y, int x) {
    uint32_t iy, cy, ix, cx;
    e.dsh.divmod((uint32_t)(y + e.ph), iy, cy);
    e.dsw.divmod((uint32_t)(x + e.pw), ix, cx);
    return (int64_t)((int)cy * e.sw + (int)cx) * e.Q * e.plane_stride + (int64_t)n * e.img_stride +
           ((int64_t)iy * e.Wc + ix) * 4;
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

}  // namespace fxb
