// Tensor-map (TMA) helpers: host-side descriptor encoding through the driver entry point that the
// CUDA runtime hands out (the library does not link against libcuda, so it still loads on a
// machine without a driver), and the device-side bulk tensor copy / mbarrier transaction wrappers.
#pragma once
#include <cuda.h>

#include <cstring>
#include <vector>

#include "fxb_common.cuh"

namespace fxb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// Returns the driver's cuTensorMapEncodeTiled, or nullptr when the driver does not offer it.
inline EncodeTiledFn tensor_map_encoder() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        else
            (void)cudaGetLastError();
    }
    return fn;
}

// f32 tensor of `rank` dimensions (innermost first), no swizzle, no interleave, out-of-bounds
// elements read as zero.  `dims` in elements, `strides_bytes[i]` = byte stride of dimension i+1
// (multiples of 16), `box` = extent of one copy per dimension (each <= 256, box[0]*4 a multiple of 16).
struct TensorMapKey {
    const void* base;
    int rank;
    uint64_t dims[5], strides[4];
    uint32_t box[5];
};
// A training loop encodes the same few dozen maps every step (fixed arena, fixed shapes); the driver call
// costs a microsecond or two each, which shows once a step is about a millisecond.  Small per-thread cache.
inline bool encode_f32_map_uncached(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                                    const uint64_t* strides_bytes, const uint32_t* box);
inline bool encode_f32_map(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                           const uint64_t* strides_bytes, const uint32_t* box) {
    if (rank < 1 || rank > 5) return false;
    struct Entry { TensorMapKey key; CUtensorMap map; };
    static thread_local std::vector<Entry> cache;
    TensorMapKey k;
    memset(&k, 0, sizeof(k));
    k.base = base; k.rank = rank;
    for (int i = 0; i < rank; ++i) { k.dims[i] = dims[i]; k.box[i] = box[i]; }
    for (int i = 0; i + 1 < rank; ++i) k.strides[i] = strides_bytes[i];
    for (const Entry& e : cache)
        if (memcmp(&e.key, &k, sizeof(k)) == 0) { *map = e.map; return true; }
    if (!encode_f32_map_uncached(map, base, rank, dims, strides_bytes, box)) return false;
    if (cache.size() >= 256) cache.clear();
    Entry e;
    e.key = k; e.map = *map;
    cache.push_back(e);
    return true;
}
inline bool encode_f32_map_uncached(CUtensorMap* map, const void* base, int rank, const uint64_t* dims,
                                    const uint64_t* strides_bytes, const uint32_t* box) {
    EncodeTiledFn enc = tensor_map_encoder();
    if (enc == nullptr || rank < 1 || rank > 5) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) return false;
    cuuint64_t gd[5];
    cuuint64_t gs[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) {
        if (dims[i] == 0 || dims[i] > 0xFFFFFFFFull || box[i] == 0 || box[i] > 256) return false;
        gd[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
    }
    if ((box[0] * 4u) % 16u != 0) return false;
    for (int i = 0; i + 1 < rank; ++i) {
        if (strides_bytes[i] % 16 != 0 || strides_bytes[i] >= (1ull << 40)) return false;
        gs[i] = strides_bytes[i];
    }
    const CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, const_cast<void*>(base), gd, gs, bx, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

#ifdef __CUDACC__
// Announces `bytes` of asynchronous copies on the barrier and counts as this thread's arrival.
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One box of a 5-D / 4-D / 3-D tensor map -> shared memory of this CTA; completion is reported to the
// mbarrier as transferred bytes.  The innermost coordinate must be a multiple of
// 4 elements (16 bytes); coordinates may lie outside the tensor (those elements read as zero).
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t smem_dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3, int c4) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
        ::"r"(smem_dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
#endif

}  // namespace fxb
