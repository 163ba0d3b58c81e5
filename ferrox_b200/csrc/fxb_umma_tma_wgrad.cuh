// f32 filter-gradient engine for sm_100a fed by the tensor-map copy engine.
//
//   dW[o][c][r][s] = sum over (n, oy, ox) of dZ[n][o][oy][ox] * X[n][c][oy*sh + r - ph][ox*sw + s - pw]
//
// as a GEMM  D[o][(tap, c)] = sum_k A[o][k] * B[(tap, c)][k]  whose contraction index k runs over
// the images and output pixels.  A 4-wide K chunk is FOUR CONSECUTIVE IMAGES at one pixel, so a
// filter tap only shifts pixel coordinates (which have no alignment rule for the copy engine) and
// one copy of the input serves every tap.  Both operands are prepared by a pre-pass, hi and lo parts:
//   A = DZN[g][oy][ox][o][4]                g = n / 4: dZ of images 4g..4g+3 at one output pixel
//   B = XN[cls][g][iy][ix][c][4]            the input in padded coordinates (y + ph, x + pw), split into
//       stride classes cls = (yp % sh, xp % sw) at (iy, ix) = (yp / sh, xp / sw); tap (r, s) pairs output
//       pixel (oy, ox) with class (r % sh, s % sw) at (oy + r / sh, ox + s / sw).  Cells in the top / left
//       padding are stored as zeros, cells beyond the bottom / right edge are out-of-bounds coordinates
//       (read as zeros), and so are the output pixels of a partial box.
// A 32-deep K stage is a box of bw x bh output pixels (bw * bh = 8) of one image group: one 5-D box per
// operand half (A) or per filter tap of the column tile (B), each landing in shared memory as
// [chunk][row][16 bytes], the canonical no-swizzle K-major UMMA layout.
//
// A column tile of 128 holds 128/Cb taps of Cb channels (Cb = min(padded C, 128)); each tap has
// its own operand sub-tile and its own N = Cb slice of the accumulator.  K is split over CTAs
// (split-K); every split writes raw partial sums that a reduction kernel adds in split order.
// Roles, accumulation scheme (3xTF32, drain every 32 values of K) and bounded waits are those of
// umma_tma_conv_kernel (here with eight drain warps, two column halves).
#pragma once
#include "fxb_umma_tma_engine.cuh"

namespace fxb {

struct TmaWgradParams {
    CUtensorMap a_hi, a_lo, b_hi, b_lo;
    int tm, tn, splits;       // items = tm * tn * splits, m fastest
    int stages_total;         // 32-deep K stages over the whole batch
    int stages_per_split;
    int three_pass;
    int K, C, RS, S;          // output channels, input channels, taps, filter width
    int Cb;                   // channels per tap sub-tile (64 or 128)
    int tpt;                  // taps per column tile (128 / Cb)
    int cblocks;              // column tiles per tap (padded C / 128, at least 1)
    int sh, sw;
    int n4;                   // image groups (images / 4, rounded up)
    int ncls;                 // stride classes (sh * sw)
    int bw, bh;               // output-pixel box of one stage, bw * bh = 8
    FastDiv dSpg, dPW;        // stage -> (image group, box row, box column)
    int drain_group;          // stages of K accumulated in TMEM before the drain warps add them into registers
    float* out;               // dW (splits == 1) or the partial-sum workspace
    int64_t split_stride;     // elements between the partial results of consecutive splits
};

template <int BN>
__global__ void __launch_bounds__(TMA_THREADS, 1)
umma_tma_wgrad_kernel(const __grid_constant__ TmaWgradParams prm, DeviceStatus* status) {
    static_assert(BN == 128, "the filter-gradient engine uses 128-wide column tiles");
    using Cfg = TmaCfg<BN>;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem);
    uint64_t* empty_bar = reinterpret_cast<uint64_t*>(smem + 64);
    uint64_t* accf_bar = reinterpret_cast<uint64_t*>(smem + 128);
    uint64_t* acce_bar = reinterpret_cast<uint64_t*>(smem + 192);
    uint64_t* corrf_bar = reinterpret_cast<uint64_t*>(smem + 256);
    uint64_t* corre_bar = reinterpret_cast<uint64_t*>(smem + 272);
    uint64_t* drain_bar = reinterpret_cast<uint64_t*>(smem + 288);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 304);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 308);
    volatile int* never_flag = reinterpret_cast<volatile int*>(smem + 312);
    uint8_t* stage_base = smem + Cfg::AUX_BYTES;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int total_items = prm.tm * prm.tn * prm.splits;
    const bool three_pass = prm.three_pass != 0;

    // item t -> (m tile, column tile, split) and its stage range
    auto item_stages = [&](int t, int& mt, int& nt, int& z, int& s_begin) -> int {
        mt = t % prm.tm;
        const int rest = t / prm.tm;
        nt = rest % prm.tn;
        z = rest / prm.tn;
        s_begin = z * prm.stages_per_split;
        int e = s_begin + prm.stages_per_split;
        if (e > prm.stages_total) e = prm.stages_total;
        return e > s_begin ? e - s_begin : 0;
    };

    if (tid == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        for (int b = 0; b < Cfg::NBUF; ++b) {
            mbar_init(smem_u32(&accf_bar[b]), 1);
            mbar_init(smem_u32(&acce_bar[b]), 8);
        }
        for (int b = 0; b < Cfg::NCORR; ++b) {
            mbar_init(smem_u32(&corrf_bar[b]), 1);
            mbar_init(smem_u32(&corre_bar[b]), 8);
        }
        mbar_init(smem_u32(drain_bar), 1);
        *abort_flag = 0;
        *never_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), Cfg::TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t sub_bytes = (uint32_t)(TMA_KCH * prm.Cb * 16);  // one tap sub-tile (hi or lo)

    if (warp == 0) {
        // ------------------------------------------------------------------ copy issue
        if (lane == 0) {
            tma_prefetch_map(&prm.a_hi);
            tma_prefetch_map(&prm.a_lo);
            tma_prefetch_map(&prm.b_hi);
            tma_prefetch_map(&prm.b_lo);
        }
        // lanes 0, 1: dZ hi, lo.  lanes 2 + 2j, 3 + 2j: X hi, lo of tap j of the column tile (j < tpt <= 8).
        const bool is_a = lane < 2;
        const bool is_lo = (lane & 1) != 0;
        const int jtap = (lane - 2) >> 1;
        const bool has_copy = (is_a || jtap < prm.tpt) && (three_pass || !is_lo);
        const uint32_t stage_tx = (uint32_t)(Cfg::A_BYTES + Cfg::B_BYTES) * (three_pass ? 2u : 1u);
        uint32_t pit = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
            int mt, nt, z, s_begin;
            const int nst = item_stages(t, mt, nt, z, s_begin);
            // column tile -> first tap and channel block
            const int tap0 = prm.cblocks > 1 ? nt / prm.cblocks : nt * prm.tpt;
            const int cblk = prm.cblocks > 1 ? nt % prm.cblocks : 0;
            // this lane's tap: stride class and window displacement
            int cls_base = prm.ncls * prm.n4, qy = 0, qx = 0;  // a tap beyond the filter reads outside the tensor: zeros
            if (!is_a && jtap < prm.tpt) {
                const int tap = tap0 + jtap;
                if (tap < prm.RS) {
                    const int r = tap / prm.S, sx = tap - r * prm.S;
                    qy = r / prm.sh;
                    qx = sx / prm.sw;
                    cls_base = ((r - qy * prm.sh) * prm.sw + (sx - qx * prm.sw)) * prm.n4;
                }
            }
            for (int sb = 0; sb < nst && ok; ++sb) {
                const int s = (int)(pit % Cfg::STAGES);
                const uint32_t ph = (pit / Cfg::STAGES) & 1u;
                const uint32_t bar = smem_u32(&full_bar[s]);
                if (lane == 0) {
                    ok = mbar_wait_bounded(smem_u32(&empty_bar[s]), ph ^ 1u, abort_flag, status, TMA_WAIT_STAGE_EMPTY);
                    if (ok) mbar_arrive_expect_tx(bar, stage_tx);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                const uint32_t a_hi = smem_u32(stage_base + (size_t)s * Cfg::STAGE_BYTES);
                const uint32_t a_lo = a_hi + Cfg::A_BYTES;
                const uint32_t b_hi = a_lo + Cfg::A_BYTES;
                const uint32_t b_lo = b_hi + Cfg::B_BYTES;
                const int stage = s_begin + sb;
                if (has_copy) {
                    uint32_t g, rem, py, px;
                    prm.dSpg.divmod((uint32_t)stage, g, rem);
                    prm.dPW.divmod(rem, py, px);
                    const int oy0 = (int)py * prm.bh, ox0 = (int)px * prm.bw;
                    if (is_a) {
                        tma_load_5d(is_lo ? a_lo : a_hi, is_lo ? &prm.a_lo : &prm.a_hi, bar, 0, mt * (UMMA_BM / 16), ox0, oy0, (int)g);
                    } else {
                        tma_load_5d((is_lo ? b_lo : b_hi) + (uint32_t)jtap * sub_bytes, is_lo ? &prm.b_lo : &prm.b_hi, bar, 0,
                                    cblk * (BN / 16), ox0 + qx, oy0 + qy, cls_base + (int)g);
                    }
                }
                ++pit;
            }
        }
        if (lane == 0) {
            const uint32_t first = pit > (uint32_t)Cfg::STAGES ? pit - Cfg::STAGES : 0u;
            for (uint32_t q = first; q < pit; ++q)
                mbar_wait_bounded(smem_u32(&full_bar[q % Cfg::STAGES]), (q / Cfg::STAGES) & 1u, never_flag, status,
                                  TMA_WAIT_COPIES, 200000000LL);
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            // instruction descriptor with N = Cb
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(prm.Cb >> 3) << 17) |
                                   ((uint32_t)(UMMA_BM >> 4) << 24);
            const uint32_t lbo_b = (uint32_t)prm.Cb * 16u;
            uint32_t sit = 0, mit = 0, tix = 0;  // stages consumed, accumulator groups issued, tiles
            const int G = prm.drain_group;
            bool ok = true;
            bool issued_any = false;
            for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
                int mt, nt, z, s_begin;
                const int nst = item_stages(t, mt, nt, z, s_begin);
                if (nst == 0) continue;
                const uint32_t cb = tix % Cfg::NCORR;
                if (three_pass) {
                    ok = mbar_wait_bounded(smem_u32(&corre_bar[cb]), ((tix / Cfg::NCORR) & 1u) ^ 1u, abort_flag, status,
                                           TMA_WAIT_CORR_EMPTY);
                    if (!ok) break;
                }
                const uint32_t d_corr = tmem_base + cb * BN;
                int in_group = 0;
                for (int sb = 0; sb < nst; ++sb) {
                    const int s = (int)(sit % Cfg::STAGES);
                    const uint32_t ph = (sit / Cfg::STAGES) & 1u;
                    const int b = (int)(mit % Cfg::NBUF);
                    ok = mbar_wait_bounded(smem_u32(&full_bar[s]), ph, abort_flag, status, TMA_WAIT_STAGE_FULL);
                    if (!ok) break;
                    if (in_group == 0) {
                        ok = mbar_wait_bounded(smem_u32(&acce_bar[b]), ((mit / Cfg::NBUF) & 1u) ^ 1u, abort_flag, status,
                                               TMA_WAIT_ACC_EMPTY);
                        if (!ok) break;
                    }
                    tc_fence_after_sync();
                    const uint32_t a_hi = smem_u32(stage_base + (size_t)s * Cfg::STAGE_BYTES);
                    const uint32_t a_lo = a_hi + Cfg::A_BYTES;
                    const uint32_t b_hi = a_lo + Cfg::A_BYTES;
                    const uint32_t b_lo = b_hi + Cfg::B_BYTES;
                    const uint32_t d_main = tmem_base + (uint32_t)(BN * (Cfg::NCORR + b));
                    for (int j = 0; j < prm.tpt; ++j) {
                        const uint32_t bj_hi = b_hi + (uint32_t)j * sub_bytes, bj_lo = b_lo + (uint32_t)j * sub_bytes;
                        const uint32_t dcol = (uint32_t)(j * prm.Cb);
#pragma unroll
                        for (int kk = 0; kk < TMA_BK / 8; ++kk) {
                            const uint32_t ao = kk * 2 * Cfg::LBO_A, bo = kk * 2 * lbo_b;
                            const uint64_t dah = umma_smem_desc(a_hi + ao, Cfg::LBO_A);
                            const uint64_t dbh = umma_smem_desc(bj_hi + bo, lbo_b);
                            if (three_pass) {
                                const uint64_t dal = umma_smem_desc(a_lo + ao, Cfg::LBO_A);
                                const uint64_t dbl = umma_smem_desc(bj_lo + bo, lbo_b);
                                umma_tf32(d_corr + dcol, dal, dbh, idesc, (sb > 0 || kk > 0) ? 1u : 0u);
                                umma_tf32(d_corr + dcol, dah, dbl, idesc, 1u);
                            }
                            umma_tf32(d_main + dcol, dah, dbh, idesc, (kk == 0 && in_group == 0) ? 0u : 1u);
                        }
                    }
                    issued_any = true;
                    umma_commit(smem_u32(&empty_bar[s]));
                    ++sit;
                    if (++in_group == G || sb == nst - 1) {
                        umma_commit(smem_u32(&accf_bar[b]));
                        ++mit;
                        in_group = 0;
                    }
                }
                if (!ok) break;
                if (three_pass) umma_commit(smem_u32(&corrf_bar[cb]));
                ++tix;
            }
            if (!ok && issued_any) {
                umma_commit(smem_u32(drain_bar));
                mbar_wait_bounded(smem_u32(drain_bar), 0u, never_flag, status, TMA_WAIT_DRAIN, 200000000LL);
            }
        }
        __syncwarp();
        tc_fence_before_sync();
    } else if (warp >= 4) {
        // ------------------------------------------------------------------ drain warps + epilogue
        const int dw = warp - 4;
        const int quad = warp & 3;
        const int half = dw >> 2;
        constexpr int DCOLS = BN / 2;
        const int cbeg = half * DCOLS;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        uint32_t git = 0, tix = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
            int mt, nt, z, s_begin;
            const int nst = item_stages(t, mt, nt, z, s_begin);
            float acc[DCOLS];
#pragma unroll
            for (int i = 0; i < DCOLS; ++i) acc[i] = 0.f;
            const int ngroups = (nst + prm.drain_group - 1) / prm.drain_group;
            for (int g = 0; g < ngroups && ok; ++g) {
                const int b = (int)(git % Cfg::NBUF);
                ok = mbar_wait_bounded(smem_u32(&accf_bar[b]), (git / Cfg::NBUF) & 1u, abort_flag, status, TMA_WAIT_ACC_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after_sync();
                {
                    uint32_t r[DCOLS];
#pragma unroll
                    for (int c = 0; c < DCOLS; c += 16)
                        tmem_ld16(tmem_base + lane_addr + (uint32_t)(BN * (Cfg::NCORR + b) + cbeg + c),
                                  *reinterpret_cast<uint32_t(*)[16]>(&r[c]));
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < DCOLS; ++i) acc[i] += __uint_as_float(r[i]);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acce_bar[b]));
                ++git;
            }
            if (ok && nst > 0) {
                if (three_pass) {
                    const uint32_t cb = tix % Cfg::NCORR;
                    ok = mbar_wait_bounded(smem_u32(&corrf_bar[cb]), (tix / Cfg::NCORR) & 1u, abort_flag, status, TMA_WAIT_CORR_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok) {
                        tc_fence_after_sync();
                        uint32_t r[DCOLS];
#pragma unroll
                        for (int c = 0; c < DCOLS; c += 16)
                            tmem_ld16(tmem_base + lane_addr + (uint32_t)(cb * BN + cbeg + c),
                                      *reinterpret_cast<uint32_t(*)[16]>(&r[c]));
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < DCOLS; ++i) acc[i] += __uint_as_float(r[i]);
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&corre_bar[cb]));
                    }
                }
                ++tix;
            }
            if (!ok) break;
            // raw partial sums: part[z][o*CRS + c*RS + tap]
            const int o = mt * UMMA_BM + quad * 32 + lane;
            if (o < prm.K) {
                const int tap0 = prm.cblocks > 1 ? nt / prm.cblocks : nt * prm.tpt;
                const int c0 = prm.cblocks > 1 ? (nt % prm.cblocks) * BN : 0;
                float* outp = prm.out + (size_t)z * prm.split_stride + (size_t)o * prm.C * prm.RS;
#pragma unroll
                for (int i = 0; i < DCOLS; ++i) {
                    const int col = cbeg + i;
                    const int j = col / prm.Cb, cc = col - j * prm.Cb;
                    const int tap = tap0 + j, c = c0 + cc;
                    if (tap < prm.RS && c < prm.C) outp[(size_t)c * prm.RS + tap] = acc[i];
                }
            }
        }
        tc_fence_before_sync();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace fxb
