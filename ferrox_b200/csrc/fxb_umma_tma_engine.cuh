// f32 convolution engine for sm_100a fed by the tensor-map copy engine (TMA).
//
// Same arithmetic as umma_contract_kernel (3xTF32 on tcgen05.mma kind::tf32, main accumulators
// drained into f32 registers every 32 values of K, long-lived correction accumulator), but the
// operand tiles are filled by cp.async.bulk.tensor copies instead of by producer threads:
//
//   * The image operand lives in hi / lo "class slabs"  S[plane][n][iy][ix][4]  (4 consecutive
//     channels per pixel; for a strided forward convolution one plane per stride-residue class,
//     so that every filter tap reads a unit-stride window).  An M tile is a patch of TW x TH
//     pixels in NI consecutive images (TW*TH*NI = 128).  For one 4-wide K chunk (tap, channel
//     slab) the patch is one box  [TW*4 floats, TH, NI images, 1 plane]  of the tensor map, and
//     it lands in shared memory as 128 rows x 16 bytes: exactly one K slab of the canonical
//     no-swizzle K-major UMMA layout (LBO = 2048).  When the channel slabs per tap are a multiple
//     of 8, the 8 chunks of a stage are 8 consecutive planes and one box of 8 planes fills the
//     whole stage.  Padding, patch overhang and the K tail are out-of-bounds coordinates, which
//     the copy engine fills with zeros.
//   * The filter operand lives chunk-major,  F[kchunk][row/16][16][4],  and one box
//     [64 floats, BN/16, 8 chunks]  fills a whole stage (LBO = BN*16).
//
// CTA = 20 warps: warp 0 issues the copies (4 or 18 per 32-wide K stage, one lane each), warp 1 lane 0
// issues the MMAs, warps 4-19 drain the accumulators and run the epilogue (bias + activation +
// store) from registers.  Nothing but the epilogue touches the load/store unit, so output stores
// do not queue behind operand traffic.  Every mbarrier wait is bounded; on expiry the status
// block records where, all roles leave, copies in flight are awaited and TMEM is released.
#pragma once
#include "fxb_tma.cuh"
#include "fxb_umma_engine.cuh"

namespace fxb {

constexpr int TMA_BK = 32;               // K per stage
constexpr int TMA_KCH = TMA_BK / 4;      // 4-wide K chunks per stage
constexpr int TMA_THREADS = 384;          // filter-gradient kernel: 4 + 8 drain warps
constexpr int TMA_CONV_THREADS = 640;     // forward / input-gradient kernel: 4 + 16 drain warps
constexpr int TMA_MAX_CLS = 4;           // stride classes that one launch can merge
constexpr int TMA_BIAS_MAX = 2048;       // bias vectors up to this length are staged in shared memory

template <int BN> struct TmaCfg {
    static constexpr int LBO_A = UMMA_BM * 16;
    static constexpr int LBO_B = BN * 16;
    static constexpr int A_BYTES = TMA_KCH * LBO_A;  // one copy (hi or lo) of a 128 x 32 tile
    static constexpr int B_BYTES = TMA_KCH * LBO_B;
    static constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES;
    static constexpr int AUX_BYTES = 1024 + TMA_BIAS_MAX * 4;  // barriers etc. + the bias vector
    static constexpr int STAGES_RAW = (227 * 1024 - AUX_BYTES) / STAGE_BYTES;
    static constexpr int STAGES = STAGES_RAW > 8 ? 8 : STAGES_RAW;
    static constexpr int SMEM_BYTES = AUX_BYTES + STAGES * STAGE_BYTES;
    static constexpr int NCORR = BN == 128 ? 1 : 2;
    static constexpr int NBUF = BN == 128 ? 3 : BN == 64 ? 6 : 3;
    static constexpr int COLS_USED = BN * (NCORR + NBUF);
    static constexpr int TMEM_COLS = COLS_USED <= 32 ? 32 : COLS_USED <= 64 ? 64 : COLS_USED <= 128 ? 128
                                     : COLS_USED <= 256 ? 256 : 512;
    static_assert(BN == 16 || BN == 64 || BN == 128, "supported tile widths");
    static_assert(COLS_USED <= 512, "TMEM has 512 columns");
    static_assert(STAGES >= 2, "at least two stages");
};

struct TmaConvParams {
    CUtensorMap a_hi, a_lo;
    CUtensorMap b_hi[TMA_MAX_CLS], b_lo[TMA_MAX_CLS];  // filter maps, one pair per merged stride class
    // work: ncls classes x tm patch tiles x tn column tiles, class fastest, then m
    int ncls;           // 1, or the stride classes of an input gradient merged into one launch
    int tm, tn;
    int ncols;          // valid columns (N of the GEMM)
    int kchunks[TMA_MAX_CLS];  // 4-wide K chunks in total (K = 4 * kchunks), per class
    int three_pass;
    // patch geometry: tile mt -> (image group g, patch row py, patch column px)
    int tw_log, th_log, ni;
    FastDiv dPP, dPW;
    // K chunk kc -> (tap, slab q) -> plane and window displacement
    FastDiv dQ, dS[TMA_MAX_CLS];
    int Q;              // channel slabs per tap
    int sh, sw;         // forward: stride (class split); input gradient: 1, 1
    int dir;            // +1 forward (window at +tap/stride), -1 input gradient (window at -tap)
    int by[TMA_MAX_CLS], bx[TMA_MAX_CLS];  // window origin offset, per class
    int planes;         // number of planes of the slab tensor (an out-of-range plane reads zeros)
    int a_chunks;       // K chunks (planes) one image copy brings: 8 (whole stage) or 1
    // output: out[img*img_stride + goff + oy*gys + ox*gxs + n*nstr] = act(acc + bias[n])
    float* out;
    const float* bias;
    int act;
    int64_t img_stride, nstr, goff[TMA_MAX_CLS], gys, gxs;
    int n_img, Hv, Wv;  // valid images and patch-grid extent
    int vec_store;      // 1: four consecutive rows are four consecutive, 16-byte aligned output floats (selects the VEC kernel)
    // split-K (forward convolutions with fewer tiles than SMs; ncls == 1): split z of a tile contracts the
    // stages [z * stages_per_split, ...) and writes raw partial sums to out + z * split_stride; bias and
    // activation are applied by the kernel that adds the splits
    int splits = 1, stages_per_split = 0;
    int64_t split_stride = 0;
    // stages of K accumulated in TMEM before the drain warps add the accumulator into their f32 registers
    int drain_group = 1;
    // GEMM use (one-pixel images): each row's columns are consecutive floats -> 16-byte stores along a row
    int row_vec = 0;
    int a_nshift = 0;   // the image coordinate of the row-operand map counts groups of 2^a_nshift rows
    // forward convolutions (ncls == 1, splits == 1): also write the activated output as the next layer's class slabs
    SlabEmit emit;
    // > 0: items walk the tiles in groups of group_m row tiles (all column tiles of a group before the next
    // group), so that CTAs running side by side share operand rows in L2.  splits == 1 only (with merged stride
    // classes the class stays the fastest index and the grouping applies to the (row tile, column tile) part).
    int group_m = 0;
};

enum : int { TMA_WAIT_STAGE_EMPTY = 11, TMA_WAIT_STAGE_FULL = 12, TMA_WAIT_ACC_FULL = 13, TMA_WAIT_DRAIN = 14,
             TMA_WAIT_ACC_EMPTY = 15, TMA_WAIT_CORR_FULL = 16, TMA_WAIT_CORR_EMPTY = 17, TMA_WAIT_COPIES = 18 };

template <int BN, bool VEC>
__global__ void __launch_bounds__(TMA_CONV_THREADS, 1)
umma_tma_conv_kernel(const __grid_constant__ TmaConvParams prm, DeviceStatus* status) {
    using Cfg = TmaCfg<BN>;
    extern __shared__ __align__(1024) uint8_t smem[];
    // aux region (bytes): [0,64) stage-full barriers, [64,128) stage-empty, [128,192) accumulator-full,
    // [192,256) accumulator-empty, [256,272) correction-full, [272,288) correction-empty, [288,296) drain,
    // [304,308) TMEM base, [308,312) abort flag, [312,316) a flag that is never raised.
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
    float* bias_s = reinterpret_cast<float*>(smem + 1024);
    uint8_t* stage_base = smem + Cfg::AUX_BYTES;

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int total_items = prm.tm * prm.tn * prm.ncls * prm.splits;
    const bool three_pass = prm.three_pass != 0;
    // item t -> (stride class, patch tile, column tile); the K length depends on the class
    // The classes have different K lengths; rotating the class with the round of the persistent loop gives
    // every CTA a mix of them (without it CTA b would always draw class b % ncls when the grid is a multiple
    // of ncls).  The rotation is constant inside a group of ncls consecutive items, so the map stays one to one.
    const int rot_ok = (gridDim.x % prm.ncls) == 0;
    auto decode = [&](int t, int& cls, int& mt, int& nt, int& z, int& s_begin) -> int {
        const int round = rot_ok ? t / (int)gridDim.x : 0;
        cls = (t + round) % prm.ncls;
        const int rest = t / prm.ncls;
        if (prm.group_m > 0) {
            const int per = prm.group_m * prm.tn;
            const int grp = rest / per, r = rest - grp * per;
            const int first = grp * prm.group_m;
            const int gsz = min(prm.group_m, prm.tm - first);
            nt = r / gsz;
            mt = first + (r - nt * gsz);
            z = 0;
        } else {
            mt = rest % prm.tm;
            const int ntz = rest / prm.tm;
            nt = ntz % prm.tn;
            z = ntz / prm.tn;
        }
        const int all = (prm.kchunks[cls] + TMA_KCH - 1) / TMA_KCH;
        if (prm.splits == 1) { s_begin = 0; return all; }
        s_begin = z * prm.stages_per_split;
        const int e = min(all, s_begin + prm.stages_per_split);
        return e > s_begin ? e - s_begin : 0;
    };
    const int TW = 1 << prm.tw_log, TH = 1 << prm.th_log;

    if (tid == 0) {
        for (int s = 0; s < Cfg::STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);   // the issuing lane's arrive.expect_tx
            mbar_init(smem_u32(&empty_bar[s]), 1);  // tcgen05.commit
        }
        for (int b = 0; b < Cfg::NBUF; ++b) {
            mbar_init(smem_u32(&accf_bar[b]), 1);
            mbar_init(smem_u32(&acce_bar[b]), 16);  // one arrival per drain warp
        }
        for (int b = 0; b < Cfg::NCORR; ++b) {
            mbar_init(smem_u32(&corrf_bar[b]), 1);
            mbar_init(smem_u32(&corre_bar[b]), 16);
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
    // The bias vector is read from shared memory in the epilogue (zeros when there is none).
    const bool bias_in_smem = prm.ncols <= TMA_BIAS_MAX;
    if (bias_in_smem)
        for (int i = tid; i < TMA_BIAS_MAX; i += TMA_CONV_THREADS)
            bias_s[i] = (prm.bias != nullptr && i < prm.ncols) ? __ldg(prm.bias + i) : 0.f;
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ copy issue
        if (lane == 0) {
            tma_prefetch_map(&prm.a_hi);
            tma_prefetch_map(&prm.a_lo);
            for (int q = 0; q < prm.ncls; ++q) {
                tma_prefetch_map(&prm.b_hi[q]);
                tma_prefetch_map(&prm.b_lo[q]);
            }
        }
        // a_chunks == 1: lane l < 16 copies image chunk (l & 7) of the hi (l < 8) or lo array;
        // a_chunks == 8: lanes 0 / 8 copy the whole stage of the hi / lo array.  Lanes 16, 17: filter hi, lo.
        const bool is_a = lane < 16;
        const bool is_lo = is_a ? lane >= 8 : lane == 17;
        const bool has_copy = (lane < 18) && (three_pass || !is_lo) && (!is_a || prm.a_chunks == 1 || (lane & 7) == 0);
        const uint32_t stage_tx = (uint32_t)(Cfg::A_BYTES + Cfg::B_BYTES) * (three_pass ? 2u : 1u);
        uint32_t pit = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
            int cls, mt, nt, z, s_begin;
            const int nstages = decode(t, cls, mt, nt, z, s_begin);
            uint32_t g, pr, py, px;
            prm.dPP.divmod((uint32_t)mt, g, pr);
            prm.dPW.divmod(pr, py, px);
            const int y_base = (int)py * TH + prm.by[cls], x_base = (int)px * TW + prm.bx[cls], n_base = (int)g * prm.ni;
            for (int sb = 0; sb < nstages && ok; ++sb) {
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
                if (has_copy) {
                    if (is_a) {
                        const int j = lane & 7;
                        const int kc = (s_begin + sb) * TMA_KCH + j;
                        uint32_t tap, q, jr, js;
                        prm.dQ.divmod((uint32_t)kc, tap, q);
                        prm.dS[cls].divmod(tap, jr, js);
                        int plane, y, x;
                        if (prm.dir > 0) {
                            const int qy = (int)jr / prm.sh, cy = (int)jr - qy * prm.sh;
                            const int qx = (int)js / prm.sw, cx = (int)js - qx * prm.sw;
                            plane = (cy * prm.sw + cx) * prm.Q + (int)q;
                            y = y_base + qy;
                            x = x_base + qx;
                        } else {
                            plane = (int)q;
                            y = y_base - (int)jr;
                            x = x_base - (int)js;
                        }
                        if (kc >= prm.kchunks[cls]) plane = prm.planes;  // K tail: zeros
                        tma_load_4d((is_lo ? a_lo : a_hi) + (uint32_t)j * Cfg::LBO_A, is_lo ? &prm.a_lo : &prm.a_hi, bar, x * 4,
                                    y, n_base >> prm.a_nshift, plane);
                    } else {
                        tma_load_3d(is_lo ? b_lo : b_hi, is_lo ? &prm.b_lo[cls] : &prm.b_hi[cls], bar, 0, nt * (BN / 16),
                                    (s_begin + sb) * TMA_KCH);
                    }
                }
                ++pit;
            }
        }
        // No copy may be in flight when the CTA exits: wait (bounded) for the stages still armed.
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
            const uint32_t idesc = umma_idesc<BN>();
            uint32_t sit = 0;  // stages consumed
            uint32_t mit = 0;  // main-accumulator groups issued
            uint32_t tix = 0;
            const int G = prm.drain_group;
            bool ok = true;
            bool issued_any = false;
            for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
                int cls, mt, nt, z, s_begin;
                const int nstages = decode(t, cls, mt, nt, z, s_begin);
                if (nstages == 0) continue;
                const uint32_t cb = tix % Cfg::NCORR;
                if (three_pass) {
                    ok = mbar_wait_bounded(smem_u32(&corre_bar[cb]), ((tix / Cfg::NCORR) & 1u) ^ 1u, abort_flag, status,
                                           TMA_WAIT_CORR_EMPTY);
                    if (!ok) break;
                }
                const uint32_t d_corr = tmem_base + cb * BN;
                int in_group = 0;
                for (int sb = 0; sb < nstages; ++sb) {
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
#pragma unroll
                    for (int kk = 0; kk < TMA_BK / 8; ++kk) {
                        const uint32_t ao = kk * 2 * Cfg::LBO_A, bo = kk * 2 * Cfg::LBO_B;
                        const uint64_t dah = umma_smem_desc(a_hi + ao, Cfg::LBO_A);
                        const uint64_t dbh = umma_smem_desc(b_hi + bo, Cfg::LBO_B);
                        if (three_pass) {
                            const uint64_t dal = umma_smem_desc(a_lo + ao, Cfg::LBO_A);
                            const uint64_t dbl = umma_smem_desc(b_lo + bo, Cfg::LBO_B);
                            umma_tf32(d_corr, dal, dbh, idesc, (sb > 0 || kk > 0) ? 1u : 0u);
                            umma_tf32(d_corr, dah, dbl, idesc, 1u);
                        }
                        umma_tf32(d_main, dah, dbh, idesc, (kk == 0 && in_group == 0) ? 0u : 1u);
                    }
                    issued_any = true;
                    umma_commit(smem_u32(&empty_bar[s]));
                    ++sit;
                    if (++in_group == G || sb == nstages - 1) {
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
        const int dw = warp - 4;    // 0..15
        const int quad = warp & 3;  // TMEM lane quadrant this warp may access
        const int part = dw >> 2;   // which quarter of the columns (sixteen drain warps: 4 lane quadrants x 4 column parts)
        constexpr int DCOLS = BN >= 64 ? BN / 4 : 16;
        const bool active = part * DCOLS < BN;
        const int cbeg = active ? part * DCOLS : 0;
        const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
        // Column rotation: register i of this warp holds tile column cbeg + ((i + rot) mod DCOLS).  CTAs
        // that run side by side write tiles whose addresses differ by large powers of two; with the same
        // column order everywhere they would all hit the same L2 slice at the same time.
        const int rot = DCOLS >= 32 ? (int)((blockIdx.x * 16u) % (unsigned)DCOLS) : 0;
        uint32_t git = 0, tix = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
            int cls, mt, nt, z, s_begin;
            const int nstages = decode(t, cls, mt, nt, z, s_begin);
            float acc[DCOLS];
#pragma unroll
            for (int i = 0; i < DCOLS; ++i) acc[i] = 0.f;
            const int ngroups = (nstages + prm.drain_group - 1) / prm.drain_group;
            for (int g = 0; g < ngroups && ok; ++g) {
                const int b = (int)(git % Cfg::NBUF);
                ok = mbar_wait_bounded(smem_u32(&accf_bar[b]), (git / Cfg::NBUF) & 1u, abort_flag, status, TMA_WAIT_ACC_FULL);
                ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld is warp-wide
                if (!ok) break;
                tc_fence_after_sync();
                if (active) {
                    // all loads of the group first, one wait, then the adds
                    uint32_t r[DCOLS];
#pragma unroll
                    for (int c = 0; c < DCOLS; c += 16)
                        tmem_ld16(tmem_base + lane_addr + (uint32_t)(BN * (Cfg::NCORR + b) + cbeg + ((c + rot) & (DCOLS - 1))),
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
            if (ok && nstages > 0) {
                if (three_pass) {
                    const uint32_t cb = tix % Cfg::NCORR;
                    ok = mbar_wait_bounded(smem_u32(&corrf_bar[cb]), (tix / Cfg::NCORR) & 1u, abort_flag, status, TMA_WAIT_CORR_FULL);
                    ok = __all_sync(0xffffffffu, ok);
                    if (ok) {
                        tc_fence_after_sync();
                        if (active) {
                            uint32_t r[DCOLS];
#pragma unroll
                            for (int c = 0; c < DCOLS; c += 16)
                                tmem_ld16(tmem_base + lane_addr + (uint32_t)(cb * BN + cbeg + ((c + rot) & (DCOLS - 1))),
                                          *reinterpret_cast<uint32_t(*)[16]>(&r[c]));
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < DCOLS; ++i) acc[i] += __uint_as_float(r[i]);
                        }
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(smem_u32(&corre_bar[cb]));
                    }
                }
                ++tix;
            }
            if (!ok) break;
            // fused epilogue from registers (overlaps the next item's main loop)
            uint32_t g, pr, py, px;
            prm.dPP.divmod((uint32_t)mt, g, pr);
            prm.dPW.divmod(pr, py, px);
            const int ml = quad * 32 + lane;
            const int ni = ml >> (prm.tw_log + prm.th_log);
            const int ty = (ml >> prm.tw_log) & (TH - 1), tx = ml & (TW - 1);
            const int img = (int)g * prm.ni + ni, oy = (int)py * TH + ty, ox = (int)px * TW + tx;
            const bool row_ok = img < prm.n_img && oy < prm.Hv && ox < prm.Wv;
            const int64_t moff = (int64_t)img * prm.img_stride + prm.goff[cls] + (int64_t)oy * prm.gys + (int64_t)ox * prm.gxs +
                                 (int64_t)z * prm.split_stride;
            const bool final_values = prm.splits == 1;  // raw partial sums otherwise
            const bool emit = prm.emit.hi != nullptr && final_values && row_ok;
            const int64_t eoff = emit ? slab_cell_offset(prm.emit, img, oy, ox) : 0;
            if (active) {
                const int j4 = lane & 3;
                // vector path: output offset of the first of this lane's group of four rows
                const int64_t moff4 = __shfl_sync(0xffffffffu, moff, lane & ~3);
                const bool ok4 = __shfl_sync(0xffffffffu, row_ok ? 1 : 0, lane & ~3) != 0;
                // bias and activation in place; identity / ReLU are two instructions per value, sigmoid and
                // tanh take a separate pass through the out-of-line function (kept off the common path)
                const bool relu = final_values && prm.act == FXB_ACT_RELU;
#pragma unroll
                for (int c = 0; c < DCOLS; c += 16) {
                    const int nb = nt * BN + cbeg + ((c + rot) & (DCOLS - 1));
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int n = nb + i;
                        const float bvi = !final_values ? 0.f
                                          : bias_in_smem ? bias_s[n < TMA_BIAS_MAX ? n : 0]
                                                         : ((prm.bias != nullptr && n < prm.ncols) ? __ldg(prm.bias + n) : 0.f);
                        const float t = acc[c + i] + bvi;
                        acc[c + i] = (relu && !(t > 0.f)) ? 0.f : t;
                    }
                }
                if (final_values && prm.act > FXB_ACT_RELU) {
#pragma unroll
                    for (int i = 0; i < DCOLS; ++i) acc[i] = act_apply_outlined<float>(acc[i], prm.act);
                }
#pragma unroll
                for (int c = 0; c < DCOLS; c += 16) {
                    const int nb = nt * BN + cbeg + ((c + rot) & (DCOLS - 1));
                    float v[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) v[i] = acc[c + i];
                    if (emit) {
#pragma unroll
                        for (int b4 = 0; b4 < 16; b4 += 4) {
                            const int n = nb + b4;
                            if (n < prm.ncols)  // channels beyond the last one of a partial chunk are zeros
                                store_split4(prm.emit.hi, prm.emit.lo, eoff + (int64_t)(n >> 2) * prm.emit.plane_stride, v[b4],
                                             n + 1 < prm.ncols ? v[b4 + 1] : 0.f, n + 2 < prm.ncols ? v[b4 + 2] : 0.f,
                                             n + 3 < prm.ncols ? v[b4 + 3] : 0.f);
                        }
                    }
                    if constexpr (VEC) {
                        // 4x4 transposes inside groups of four lanes (= four consecutive output floats):
                        // afterwards lane j of a group holds the four rows of column 4b+j -> one 16-byte store.
#pragma unroll
                        for (int b4 = 0; b4 < 16; b4 += 4) {
                            const bool odd = (j4 & 1) != 0, up = (j4 & 2) != 0;
                            float r0 = __shfl_xor_sync(0xffffffffu, odd ? v[b4 + 0] : v[b4 + 1], 1);
                            float r1 = __shfl_xor_sync(0xffffffffu, odd ? v[b4 + 2] : v[b4 + 3], 1);
                            if (odd) { v[b4 + 0] = r0; v[b4 + 2] = r1; } else { v[b4 + 1] = r0; v[b4 + 3] = r1; }
                            r0 = __shfl_xor_sync(0xffffffffu, up ? v[b4 + 0] : v[b4 + 2], 2);
                            r1 = __shfl_xor_sync(0xffffffffu, up ? v[b4 + 1] : v[b4 + 3], 2);
                            if (up) { v[b4 + 0] = r0; v[b4 + 1] = r1; } else { v[b4 + 2] = r0; v[b4 + 3] = r1; }
                            const int n = nb + b4 + j4;
                            if (ok4 && n < prm.ncols)
                                *reinterpret_cast<float4*>(prm.out + moff4 + (int64_t)n * prm.nstr) =
                                    make_float4(v[b4 + 0], v[b4 + 1], v[b4 + 2], v[b4 + 3]);
                        }
                    } else {
                        if (row_ok) {
                            if (prm.row_vec) {
#pragma unroll
                                for (int i = 0; i < 16; i += 4) {
                                    const int n = nb + i;
                                    if (n < prm.ncols)
                                        *reinterpret_cast<float4*>(prm.out + moff + n) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 16; ++i) {
                                    const int n = nb + i;
                                    if (n < prm.ncols) prm.out[moff + (int64_t)n * prm.nstr] = v[i];
                                }
                            }
                        }
                    }
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
