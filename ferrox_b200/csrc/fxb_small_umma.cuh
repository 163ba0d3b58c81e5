// Filter gradient of convolutions with a handful of input values per output (C*R*S <= 31, up to 64 output
// channels: the RGB first layer) on the tensor cores.
//
//   part[cta][o][k] = sum over this CTA's pixels of dZ[pixel][o] * im2col[pixel][k],   dZ = dY * act'(Y)
//
// is a GEMM with M = output channels, N = 32 im2col columns and K = pixels.  Both operands are K-major in
// memory already: four consecutive pixels of one channel are 16 contiguous bytes of dY (NCHW), i.e. one chunk of
// the no-swizzle canonical shared-memory layout [chunk][row][16 B].  Twenty-four warps stage 32-pixel K stages
// (16-byte loads of dY and Y, activation factor, hi/lo split, 16-byte stores; the im2col chunks are gathered),
// one thread issues tcgen05.mma kind::tf32 (3xTF32: hi*hi into alternating main accumulators, the two cross
// terms into a correction accumulator), four warps add the main accumulator into f32 registers every four
// stages (the tensor core's accumulation truncates) and write the CTA's partial sums at the end; the existing
// finish kernels add the partials of all CTAs in a fixed order.  Column 31 of the im2col operand is all ones,
// so that row o of the product also carries sum(dZ[.][o]) = the bias gradient.
#pragma once
#include "fxb_common.cuh"
#include "fxb_small.cuh"
#include "fxb_umma_engine.cuh"

namespace fxb {

constexpr int FLW_STAGES = 2;                    // operand stages (four measured the same)
constexpr int FLW_BK = 32;                       // pixels per stage
constexpr int FLW_KCH = FLW_BK / 4;              // 16-byte chunks per row and stage
constexpr int FLW_LBO_A = 128 * 16 + 16;         // chunk pitch (bytes); the extra 16 bytes spread the chunks of
constexpr int FLW_LBO_B = 32 * 16 + 16;          //   one row over different banks for the staging stores
constexpr int FLW_A_BYTES = FLW_KCH * FLW_LBO_A;
constexpr int FLW_B_BYTES = FLW_KCH * FLW_LBO_B;
constexpr int FLW_STAGE_BYTES = 2 * FLW_A_BYTES + 2 * FLW_B_BYTES;
constexpr int FLW_AUX_BYTES = 1024;
// Landing ring of the dY / Y loads: FLW_RING tiles, per tile and tensor one 16-byte cell per loading thread
// (asynchronous copies, 8 tiles x 16 KB in flight per SM, no registers held while they fly).  Measured: the ring
// and a four-tile register prefetch run equally fast, because the kernel is bound by the hand-offs of its short
// stages, not by memory (without any global load it takes 218 us instead of 247 us per call at batch 1024).
constexpr int FLW_RING = 8;
constexpr int FLW_RING_BYTES = FLW_RING * 2 * 512 * 16;
constexpr int FLW_SMEM_BYTES = FLW_AUX_BYTES + FLW_STAGES * FLW_STAGE_BYTES + FLW_RING_BYTES;
constexpr int FLW_A_STAGERS = 512;               // warps 0-15: one dZ chunk (dY and Y) per thread and stage
constexpr int FLW_B_STAGERS = 256;               // warps 16-23: one im2col chunk per thread and stage
constexpr int FLW_STAGERS = FLW_A_STAGERS + FLW_B_STAGERS;
constexpr int FLW_MMA_WARP = FLW_STAGERS / 32;
constexpr int FLW_THREADS = FLW_STAGERS + 32 + 128;  // + the MMA warp + four drain warps
constexpr int FLW_PREFETCH = 4;                  // tiles of gathered loads in flight per im2col staging thread
constexpr int FLW_GROUP = 4;                     // stages accumulated in TMEM between two drains
constexpr int FLW_TMEM_COLS = 128;               // correction (32) + two main accumulators (32 each)

enum : int { FLW_WAIT_STAGE_EMPTY = 31, FLW_WAIT_STAGE_FULL = 32, FLW_WAIT_ACC_FULL = 33, FLW_WAIT_ACC_EMPTY = 34,
             FLW_WAIT_CORR_FULL = 35, FLW_WAIT_DRAIN = 36 };

// Requirements (checked by the host): f32, K <= 64, C*R*S <= 31, P % 4 == 0, OW % 4 == 0, dY / Y 16-byte aligned.
__global__ void __launch_bounds__(FLW_THREADS, 1)
firstlayer_wgrad_umma_kernel(const float* __restrict__ x, const float* __restrict__ dy, const float* __restrict__ yact,
                             float* __restrict__ part, float* __restrict__ dbpart, ConvGeom g, int64_t npix, int act,
                             int sig_math, int three_pass, DeviceStatus* status) {
    extern __shared__ __align__(1024) uint8_t smem[];
    // aux region: [0,32) stage-full barriers, [32,64) stage-empty, [64,80) accumulator-full, [80,96) accumulator-empty,
    // [96,104) correction-full, [104,112) drain, [112,116) TMEM base, [116,120) abort flag, [120,124) never raised
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty_bar = reinterpret_cast<uint64_t*>(smem + 32);
    uint64_t* accf_bar = reinterpret_cast<uint64_t*>(smem + 64);
    uint64_t* acce_bar = reinterpret_cast<uint64_t*>(smem + 80);
    uint64_t* corrf_bar = reinterpret_cast<uint64_t*>(smem + 96);
    uint64_t* drain_bar = reinterpret_cast<uint64_t*>(smem + 104);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 112);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 116);
    volatile int* never_flag = reinterpret_cast<volatile int*>(smem + 120);
    uint8_t* stage_base = smem + FLW_AUX_BYTES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t ntiles = (npix + FLW_BK - 1) / FLW_BK;
    // this CTA's stages: a contiguous run of tiles (consecutive 128-byte pieces of every channel row, so that one
    // SM's requests walk through DRAM pages instead of touching a new page per request)
    const int64_t per_cta = (ntiles + gridDim.x - 1) / gridDim.x;
    const int64_t first_tile = (int64_t)blockIdx.x * per_cta;
    const int nst = (int)max((int64_t)0, min(per_cta, ntiles - first_tile));
    const int ngroups = (nst + FLW_GROUP - 1) / FLW_GROUP;

    if (tid == 0) {
        for (int s = 0; s < FLW_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), FLW_STAGERS / 32);  // one arrival per staging warp (24)
            mbar_init(smem_u32(&empty_bar[s]), 1);                // tcgen05.commit
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&accf_bar[b]), 1);
            mbar_init(smem_u32(&acce_bar[b]), 4);                 // one arrival per drain warp
        }
        mbar_init(smem_u32(corrf_bar), 1);
        mbar_init(smem_u32(drain_bar), 1);
        *abort_flag = 0;
        *never_flag = 0;
        mbar_init_fence();
    }
    if (warp == FLW_MMA_WARP) {
        tmem_alloc(smem_u32(tmem_slot), FLW_TMEM_COLS);
        tmem_relinquish();
    }
    // Rows of the dZ operand that no staging thread writes (channels 64..127) stay zero for the whole kernel.
    if (tid < FLW_A_STAGERS) {
        for (int e = tid; e < FLW_STAGES * 2 * FLW_KCH * 64; e += FLW_A_STAGERS) {
            const int row = 64 + (e & 63), kc = (e >> 6) % FLW_KCH, half = (e >> 6) / FLW_KCH % 2, s = (e >> 6) / (2 * FLW_KCH);
            *reinterpret_cast<uint4*>(stage_base + (size_t)s * FLW_STAGE_BYTES + half * FLW_A_BYTES + kc * FLW_LBO_A + row * 16) =
                make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    // Staging: sixteen warps bring in dY / Y (one 16-byte chunk of each per thread and stage), eight more gather the
    // im2col chunks (twenty-four staging warps measured 15 % faster than eight doing the same work).
    const auto tile_of = [&](int i) { return first_tile + i; };
    const auto stage_ready = [&](int i, bool& ok) -> int {  // waits until stage i's buffer is free; returns its index
        const int s = i % FLW_STAGES;
        const uint32_t ph = (uint32_t)(i / FLW_STAGES) & 1u;
        ok = mbar_wait_bounded(smem_u32(&empty_bar[s]), ph ^ 1u, abort_flag, status, FLW_WAIT_STAGE_EMPTY);
        return s;
    };
    const auto stage_done = [&](int s) {
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&full_bar[s]));
    };
    if (tid < FLW_A_STAGERS) {
        // ------------------------------------------------------------------ dZ staging: chunk kc of channel o
        // Every thread copies its own 16 bytes of dY and of Y per tile into its own cells of the landing ring
        // (cp.async, FLW_RING tiles ahead) and reads them back itself, so the ring needs no barrier.
        const int kc = tid & 7, o = tid >> 3;
        uint8_t* ring = stage_base + (size_t)FLW_STAGES * FLW_STAGE_BYTES;
        auto cell = [&](int i, int tensor) { return ring + ((size_t)((i % FLW_RING) * 2 + tensor) * 512 + tid) * 16; };
        auto fetch = [&](int i) {  // always commits one group, so that group counting stays uniform
            if (i < nst) {
                const int64_t pix = tile_of(i) * FLW_BK + kc * 4;
                const bool in = pix < npix && o < g.K;  // (npix is a multiple of 4: a chunk is inside or outside as a whole)
                uint32_t n = 0, p = 0;
                if (in) g.dP.divmod((uint32_t)pix, n, p);
                const int64_t src = ((int64_t)n * g.K + o) * g.P + p;
                cp_async16_cg(smem_u32(cell(i, 0)), dy + src, in);
                if (yact) cp_async16_cg(smem_u32(cell(i, 1)), yact + src, in);
            }
            cp_async_commit();
        };
        for (int u = 0; u < FLW_RING; ++u) fetch(u);
        bool ok = true;
        for (int i = 0; i < nst && ok; ++i) {
            cp_async_wait_group<FLW_RING - 1>();  // tile i has landed (this thread's cells)
            float4 v = *reinterpret_cast<const float4*>(cell(i, 0));
            if (yact) {
                const float4 a = *reinterpret_cast<const float4*>(cell(i, 1));
                v.x *= act_grad_factor<float>(a.x, act, sig_math);
                v.y *= act_grad_factor<float>(a.y, act, sig_math);
                v.z *= act_grad_factor<float>(a.z, act, sig_math);
                v.w *= act_grad_factor<float>(a.w, act, sig_math);
            }
            fetch(i + FLW_RING);  // the cells just read are free again
            const int s = stage_ready(i, ok);
            if (!ok) break;
            uint8_t* a_hi = stage_base + (size_t)s * FLW_STAGE_BYTES;
            const int off = kc * FLW_LBO_A + o * 16;
            store_split4(reinterpret_cast<float*>(a_hi + off), reinterpret_cast<float*>(a_hi + FLW_A_BYTES + off), 0, v.x, v.y, v.z,
                         v.w);
            stage_done(s);
        }
        cp_async_wait_group<0>();  // no copy may be in flight when the CTA exits
    } else if (tid < FLW_STAGERS) {
        // ------------------------------------------------------------------ im2col staging: chunk kc of column r0
        const int t2 = tid - FLW_A_STAGERS;
        const int kc = t2 & 7, r0 = t2 >> 3;
        const SmallcTap tap = smallc_tap(g, r0);
        const bool ones = r0 == SMALLC_K - 1;  // the bias-gradient column (C*R*S <= 31, so it is not a real tap)
        float rx[FLW_PREFETCH][4];
        auto fetch = [&](int64_t tile, float (&xv)[4]) {
            const int64_t pix = tile * FLW_BK + kc * 4;
            const bool pin = pix < npix;
            uint32_t n = 0, p = 0, oy = 0, ox = 0;
            if (pin) {
                g.dP.divmod((uint32_t)pix, n, p);
                g.dOW.divmod(p, oy, ox);
            }
            const int y = (int)oy * g.sh - g.ph + tap.r;
            const bool row_in = pin && tap.valid && (unsigned)y < (unsigned)g.H;
            const float* xr = x + (int64_t)n * g.C * g.HW + ((int64_t)oy * g.sh - g.ph) * g.W + tap.off;
#pragma unroll
            for (int e = 0; e < 4; ++e) {  // four consecutive output pixels of one row (OW % 4 == 0)
                const int xx = ((int)ox + e) * g.sw - g.pw;
                xv[e] = (row_in && (unsigned)(xx + tap.s) < (unsigned)g.W) ? __ldg(xr + xx) : 0.f;
            }
            if (ones) xv[0] = xv[1] = xv[2] = xv[3] = pin ? 1.f : 0.f;
        };
#pragma unroll
        for (int u = 0; u < FLW_PREFETCH; ++u)
            if (u < nst) fetch(tile_of(u), rx[u]);
        bool ok = true;
        for (int i0 = 0; i0 < nst && ok; i0 += FLW_PREFETCH) {
#pragma unroll
            for (int u = 0; u < FLW_PREFETCH; ++u) {
                const int i = i0 + u;
                if (i < nst && ok) {
                    const int s = stage_ready(i, ok);
                    if (!ok) break;
                    uint8_t* b_hi = stage_base + (size_t)s * FLW_STAGE_BYTES + 2 * FLW_A_BYTES;
                    const int off = kc * FLW_LBO_B + r0 * 16;
                    store_split4(reinterpret_cast<float*>(b_hi + off), reinterpret_cast<float*>(b_hi + FLW_B_BYTES + off), 0, rx[u][0],
                                 rx[u][1], rx[u][2], rx[u][3]);
                    stage_done(s);
                    if (i + FLW_PREFETCH < nst) fetch(tile_of(i + FLW_PREFETCH), rx[u]);
                }
            }
        }
    } else if (warp == FLW_MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc<32>();
            const uint32_t d_corr = tmem_base;
            bool ok = true, issued_any = false;
            for (int i = 0; i < nst && ok; ++i) {
                const int s = i % FLW_STAGES;
                const uint32_t ph = (uint32_t)(i / FLW_STAGES) & 1u;
                const int grp = i / FLW_GROUP, b = grp & 1;
                const bool group_first = (i % FLW_GROUP) == 0, group_last = (i % FLW_GROUP) == FLW_GROUP - 1 || i == nst - 1;
                ok = mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abort_flag, status, FLW_WAIT_STAGE_FULL);
                if (!ok) break;
                if (group_first) {
                    ok = mbar_wait_bounded(smem_u32(&acce_bar[b]), ((uint32_t)(grp >> 1) & 1u) ^ 1u, abort_flag, status,
                                           FLW_WAIT_ACC_EMPTY);
                    if (!ok) break;
                }
                tc_fence_after_sync();
                const uint32_t a_hi = smem_u32(stage_base + (size_t)s * FLW_STAGE_BYTES);
                const uint32_t a_lo = a_hi + FLW_A_BYTES;
                const uint32_t b_hi = a_lo + FLW_A_BYTES;
                const uint32_t b_lo = b_hi + FLW_B_BYTES;
                const uint32_t d_main = tmem_base + 32u * (uint32_t)(1 + b);
#pragma unroll
                for (int kk = 0; kk < FLW_BK / 8; ++kk) {
                    const uint32_t ao = kk * 2 * FLW_LBO_A, bo = kk * 2 * FLW_LBO_B;
                    const uint64_t dah = umma_smem_desc(a_hi + ao, FLW_LBO_A), dal = umma_smem_desc(a_lo + ao, FLW_LBO_A);
                    const uint64_t dbh = umma_smem_desc(b_hi + bo, FLW_LBO_B), dbl = umma_smem_desc(b_lo + bo, FLW_LBO_B);
                    if (three_pass) {
                        umma_tf32(d_corr, dal, dbh, idesc, (i > 0 || kk > 0) ? 1u : 0u);
                        umma_tf32(d_corr, dah, dbl, idesc, 1u);
                    }
                    umma_tf32(d_main, dah, dbh, idesc, (group_first && kk == 0) ? 0u : 1u);
                }
                issued_any = true;
                umma_commit(smem_u32(&empty_bar[s]));
                if (group_last) umma_commit(smem_u32(&accf_bar[b]));
            }
            if (ok && nst > 0 && three_pass) umma_commit(smem_u32(corrf_bar));
            if (!ok && issued_any) {  // nothing may still be running on the tensor core when TMEM is freed
                umma_commit(smem_u32(drain_bar));
                mbar_wait_bounded(smem_u32(drain_bar), 0u, never_flag, status, FLW_WAIT_DRAIN, 200000000LL);
            }
        }
        __syncwarp();
        tc_fence_before_sync();
    } else {
        // ------------------------------------------------------------------ drain warps
        const int quad = warp & 3;  // the TMEM lane quadrant this warp may read
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.f;
        bool ok = true;
        for (int grp = 0; grp < ngroups && ok; ++grp) {
            const int b = grp & 1;
            ok = mbar_wait_bounded(smem_u32(&accf_bar[b]), (uint32_t)(grp >> 1) & 1u, abort_flag, status, FLW_WAIT_ACC_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
#pragma unroll
            for (int h = 0; h < 2; ++h) {  // 16 columns at a time (register budget of a 928-thread CTA)
                uint32_t r[16];
                tmem_ld16(tmem_base + lane_addr + 32u * (uint32_t)(1 + b) + 16u * h, r);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 16; ++i) acc[16 * h + i] += __uint_as_float(r[i]);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acce_bar[b]));
        }
        if (ok && nst > 0 && three_pass) {
            ok = mbar_wait_bounded(smem_u32(corrf_bar), 0u, abort_flag, status, FLW_WAIT_CORR_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (ok) {
                tc_fence_after_sync();
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t r[16];
                    tmem_ld16(tmem_base + lane_addr + 16u * h, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[16 * h + i] += __uint_as_float(r[i]);
                }
                tc_fence_before_sync();
            }
        }
        const int o = quad * 32 + lane;
        if (ok && o < 64) {
            float* pr = part + ((int64_t)blockIdx.x * 64 + o) * SMALLC_K;
#pragma unroll
            for (int i = 0; i < 32; i += 4) *reinterpret_cast<float4*>(pr + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
            if (dbpart != nullptr) dbpart[(int64_t)blockIdx.x * 64 + o] = acc[SMALLC_K - 1];
        }
    }
    __syncthreads();
    if (warp == FLW_MMA_WARP) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, FLW_TMEM_COLS);
    }
}

}  // namespace fxb
