// Shared-memory barriers and TMA tile loads (cp.async.bulk.tensor), as the kernels that
// stage operands through shared memory use them.  Every wait is bounded: it returns
// false when it ran out, and the caller records that and winds down.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

static constexpr uint32_t SIB_WAIT_LIMIT = 1u << 22;   // tries per wait before a block gives up

__device__ __forceinline__ uint32_t sib_smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void sib_mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(sib_smem_u32(bar)), "r"(count));
}
// Makes freshly initialised barriers visible to the copy engine.
__device__ __forceinline__ void sib_mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
}
__device__ __forceinline__ void sib_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(sib_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void sib_mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(sib_smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// Bounded wait for the phase with the given parity; false if it ran out.
__device__ __forceinline__ bool sib_mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = sib_smem_u32(bar);
    for (uint32_t i = 0; i < SIB_WAIT_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// One box of a 2-d tensor map into this block's shared memory; the bytes count towards
// `bar`.  c0 is the coordinate along the contiguous dimension: c0 * element size must be
// a multiple of 16 bytes.  The map covers this GPU's memory only; no multicast.
__device__ __forceinline__ void sib_tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n" ::"r"(sib_smem_u32(dst)),
        "l"(map), "r"(sib_smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}

// One box of a 3-d tensor map (c0 along the contiguous dimension, as above).
__device__ __forceinline__ void sib_tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(sib_smem_u32(dst)),
        "l"(map), "r"(sib_smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*SibEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                     const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                     const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
SibEncodeTiledFn sib_encode_tiled_fn();   // null if the driver does not offer it (runtime.cu)

// A map over a row-major bfloat16 matrix [rows, cols] with `row_stride` elements between
// rows: boxes of box_rows x 64 elements (128 bytes), 128-byte swizzle, zeros outside.
int sib_make_bf16_map(CUtensorMap* map, const void* base, long long rows, long long cols,
                      long long row_stride, int box_rows, const char* who);

// The same matrix (cols a multiple of 64) seen as [cols / 64][rows][64]: a box takes
// box_tiles 64-wide blocks of k of box_rows rows, laid out [block of k][row][64] in shared
// memory, so that one copy brings box_tiles * 128 contiguous bytes of every row.
int sib_make_bf16_map_k_tiles(CUtensorMap* map, const void* base, long long rows, long long cols,
                              long long row_stride, int box_rows, int box_tiles, const char* who);
