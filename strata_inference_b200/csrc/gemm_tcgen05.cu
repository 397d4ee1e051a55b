// y[R, N] = x[R, K] . W[N, K]^T on the fifth-generation tensor cores: TMA loads
// into 128-byte-swizzled shared memory, tcgen05.mma issued by one thread with
// the accumulator in tensor memory, tcgen05.ld for the epilogue.
//
// The weight rows are the M side of the instruction (a block owns 128 of them),
// the activation rows the N side (BN = 32 ... 256 of them), so the same kernel
// serves a few dozen rows (decoding large batches: every weight streamed once)
// and thousands (prompts).  The accumulator tile is therefore y transposed:
// tensor-memory lane i is weight row n0 + i, column j is activation row r0 + j.
//
//   warp 0      one lane issues the TMA loads of a STAGES-deep ring of k-blocks
//   warp 1      allocates tensor memory; one lane issues the MMAs and the commits
//   warps 2-5   epilogue: each reads its quarter of the lanes, applies the
//               epilogue (none / soft cap / gated tanh-GELU over weight rows that
//               come as 8 gate rows followed by their 8 up rows) and stores y
//
// Every wait on an mbarrier is bounded; a wait that runs out sets *error_flag,
// and the block still frees its tensor memory before it returns.
// Plain counterpart: tests/plain_gemma2.py (x @ W.T), gelu_tanh().
// Reference: src/model/layer.rs:22-43 (x . W^T), src/backend/cuda/mod.rs:828-905
// (cublasSgemm for every product).
#include <cuda.h>

#include "common.cuh"

enum { GEMM_EPI_NONE = 0, GEMM_EPI_SOFTCAP = 1, GEMM_EPI_GEGLU = 2 };

static constexpr int BM = 128;        // weight rows per block
static constexpr int BK = 64;         // k per stage: 128 bytes, one swizzle row
static constexpr int UMMA_K = 16;
static constexpr uint32_t WAIT_LIMIT = 1u << 22;   // tries per wait before a block gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// Bounded wait for the phase with the given parity; false if it ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
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
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
        : "memory");
}
// Shared-memory operand descriptor: K-major tile of rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;                    // leading byte offset (unused with this swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;          // stride between 8-row groups
    d |= (uint64_t)1 << 46;                    // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                    // 128-byte swizzle
    return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}

__device__ __forceinline__ float gemm_gelu_tanh(float g) {
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
}

struct GemmArgs {
    void* y;
    int* error_flag;
    int R, N, K;
    int y_stride;
    int epilogue;
    float cap;
};

template <int BN, int STAGES, typename OutT>
__global__ void __launch_bounds__(192)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    GemmArgs p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;
    // tiles first (1024-byte aligned), then the barriers
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * (A_BYTES + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* acc_ready = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_ready + 1);
    int* failed = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BM, r0 = blockIdx.y * BN;
    const int k_blocks = (p.K + BK - 1) / BK;
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_ready, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < k_blocks; ++kb) {
                const int s = kb % STAGES;
                const uint32_t round = kb / STAGES;
                if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1)) { *failed = 1; break; }
                mbar_arrive_expect_tx(&full[s], A_BYTES + B_BYTES);
                unsigned char* a = tiles + s * (A_BYTES + B_BYTES);
                tma_load_2d(a, &map_w, &full[s], kb * BK, n0);
                tma_load_2d(a + A_BYTES, &map_x, &full[s], kb * BK, r0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction: f32 accumulate, bf16 x bf16, both operands K-major, N = BN, M = 128
            constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) |
                                       ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            bool ok = true;
            for (int kb = 0; kb < k_blocks && ok; ++kb) {
                const int s = kb % STAGES;
                if (!mbar_wait(&full[s], (kb / STAGES) & 1)) { *failed = 2; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                unsigned char* a = tiles + s * (A_BYTES + B_BYTES);
                const uint64_t da = umma_desc(a), db = umma_desc(a + A_BYTES);
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    // 16 k = 32 bytes further along the swizzled row: + 2 in the address field
                    umma_bf16(tmem, da + 2 * k, db + 2 * k, IDESC, (kb > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(&empty[s]);      // the stage is free once these MMAs have read it
            }
            umma_commit(acc_ready);          // all MMAs done: the accumulator can be read
        }
    } else {
        // epilogue warps 2..5 own lane quarters 2, 3, 0, 1
        const int quarter = warp & 3;
        const bool ok = mbar_wait(acc_ready, 0);
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        if (!ok) {
            if (lane == 0) *failed = 3;
        } else {
            const int n = n0 + 32 * quarter + lane;             // this lane's weight row
            OutT* y = (OutT*)p.y;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(32 * quarter) << 16) + (uint32_t)c0, v);
                if (r0 + c0 >= p.R) continue;
                if (p.epilogue == GEMM_EPI_GEGLU) {
                    // rows come as 8 gates then their 8 ups: the up value sits 8 lanes on
                    const bool is_gate = (n & 15) < 8;
                    const int col = (n >> 4) * 8 + (n & 7);
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const float mine = __uint_as_float(v[j]);
                        const float up = __shfl_down_sync(0xffffffffu, mine, 8);
                        const int r = r0 + c0 + j;
                        if (is_gate && n + 8 < p.N && r < p.R)
                            y[(size_t)r * p.y_stride + col] = from_f32<OutT>(gemm_gelu_tanh(mine) * up);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        float o = __uint_as_float(v[j]);
                        if (p.epilogue == GEMM_EPI_SOFTCAP) o = p.cap * tanhf(o / p.cap);
                        const int r = r0 + c0 + j;
                        if (n < p.N && r < p.R) y[(size_t)r * p.y_stride + n] = from_f32<OutT>(o);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem),
                     "r"(TMEM_COLS)
                     : "memory");
    }
    if (threadIdx.x == 0 && *failed) atomicExch(p.error_flag, *failed);
}

// ---------------------------------------------------------------------------
// The same product for many activation rows, on pairs of SMs.
//
// A cluster of two blocks owns a tile of 256 activation rows x 256 weight rows and
// walks the tiles pair_index, pair_index + pairs, ... (persistent).  The activation
// rows are the M side here: each block of the pair holds its 128 rows of x and HALF
// of the 256 weight rows per k-block in shared memory, and one thread of the first
// block issues tcgen05.mma.cta_group::2 (M = 256, N = 256), which reads both blocks'
// halves: every byte of x and W crosses from L2 once per pair, not once per SM.
// Tensor memory holds two accumulators of 256 columns, so the epilogue warps drain
// tile i (lane = activation row, 32 consecutive outputs per tcgen05.ld: 64-byte
// stores) while the MMAs of tile i + 1 run.
//
//   warp 0      TMA loads of this block's operand halves into a ring of PAIR_STAGES;
//               the transaction bytes of both blocks are counted on the first
//               block's barrier (cp.async.bulk.tensor ... .cta_group::2)
//   warp 1      allocates tensor memory (both blocks); in the first block one lane
//               issues the MMAs; commits are multicast to both blocks' barriers
//   warps 2-5   epilogue; the second block's warps report a drained accumulator to
//               the first block's barrier
// Every mbarrier wait is bounded; both blocks meet at a cluster barrier before they
// free their tensor memory and leave.
// ---------------------------------------------------------------------------
static constexpr int PAIR_BN = 256;        // weight rows per tile (128 per block in shared memory)
static constexpr int PAIR_STAGES = 6;

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// the shared::cluster address of `p`'s counterpart in the pair's first block
__device__ __forceinline__ uint32_t in_first_block(const void* p) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, 0;\n" : "=r"(a) : "r"(smem_u32(p)));
    return a;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// the load lands in this block's shared memory; its bytes are counted on the barrier at
// the same offset in the pair's first block
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                 int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4}], [%2];\n" ::"r"(smem_u32(dst)),
        "l"(map), "r"(in_first_block(bar)), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc,
                                               uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives, once the MMAs issued so far have run, on the barrier at this offset in both blocks
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
        "[%0], %1;\n" ::"r"(smem_u32(bar)),
        "h"((uint16_t)3)
        : "memory");
}
// arrive on the barrier at this offset in the pair's first block
__device__ __forceinline__ void mbar_arrive_first_block(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(in_first_block(bar))
                 : "memory");
}

template <typename OutT>
__device__ __forceinline__ void store_run(OutT* dst, const float (&o)[32], int count);
// `count` of 32 consecutive outputs (count < 32 at the edge of the matrix)
template <>
__device__ __forceinline__ void store_run<__nv_bfloat16>(__nv_bfloat16* dst, const float (&o)[32],
                                                         int count) {
    if (count == 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __nv_bfloat162 v = __floats2bfloat162_rn(o[8 * q + 2 * k], o[8 * q + 2 * k + 1]);
                w[k] = *reinterpret_cast<const uint32_t*>(&v);
            }
            *reinterpret_cast<uint4*>(dst + 8 * q) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < count) dst[j] = __float2bfloat16(o[j]);
    }
}
template <>
__device__ __forceinline__ void store_run<float>(float* dst, const float (&o)[32], int count) {
    if (count == 32 && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
        for (int q = 0; q < 8; ++q)
            *reinterpret_cast<float4*>(dst + 4 * q) = make_float4(o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j)
            if (j < count) dst[j] = o[j];
    }
}

template <typename OutT>
__global__ void __launch_bounds__(192)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                         GemmArgs p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    constexpr uint32_t A_BYTES = 128 * BK * 2, B_BYTES = (PAIR_BN / 2) * BK * 2;
    constexpr uint32_t STAGE = A_BYTES + B_BYTES;
    unsigned char* tiles = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + PAIR_STAGES * STAGE);   // used in the first block
    uint64_t* empty = full + PAIR_STAGES;
    uint64_t* acc_full = empty + PAIR_STAGES;        // [2]
    uint64_t* acc_empty = acc_full + 2;              // [2], used in the first block
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    int* failed = reinterpret_cast<int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int tiles_m = (p.R + 255) / 256, tiles_n = (p.N + PAIR_BN - 1) / PAIR_BN;
    const int n_tiles = tiles_m * tiles_n;
    const int k_blocks = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&acc_full[b], 1);
            mbar_init(&acc_empty[b], 8);             // 4 epilogue warps of each block
        }
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(512)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();          // both blocks' barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;     // k-blocks loaded so far
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += pairs) {
                const int m0 = (tile % tiles_m) * 256 + 128 * (int)rank;
                const int n0 = (tile / tiles_m) * PAIR_BN + (PAIR_BN / 2) * (int)rank;
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    const uint32_t round = it / PAIR_STAGES;
                    if (round > 0 && !mbar_wait(&empty[s], (round - 1) & 1)) { *failed = 1; ok = false; break; }
                    if (rank == 0) mbar_arrive_expect_tx(&full[s], 2 * STAGE);
                    unsigned char* a = tiles + s * STAGE;
                    tma_load_2d_pair(a, &map_x, &full[s], kb * BK, m0);
                    tma_load_2d_pair(a + A_BYTES, &map_w, &full[s], kb * BK, n0);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // f32 accumulate, bf16 x bf16, both operands K-major, N = 256, M = 256 over the pair
            constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) |
                                       ((uint32_t)(PAIR_BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            uint32_t it = 0, done = 0;
            bool ok = true;
            for (int tile = pair; tile < n_tiles && ok; tile += pairs, ++done) {
                const uint32_t b = done & 1;
                // the epilogue of the tile two back has drained this accumulator
                if (done >= 2 && !mbar_wait(&acc_empty[b], ((done >> 1) - 1) & 1)) { *failed = 4; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const int s = it % PAIR_STAGES;
                    if (!mbar_wait(&full[s], (it / PAIR_STAGES) & 1)) { *failed = 2; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    unsigned char* a = tiles + s * STAGE;
                    const uint64_t da = umma_desc(a), db = umma_desc(a + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16_pair(tmem + 256 * b, da + 2 * k, db + 2 * k, IDESC,
                                       (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit_pair(&empty[s]);
                }
                if (ok) umma_commit_pair(&acc_full[b]);
            }
            if (!ok) {     // let nobody wait for what will not come
                umma_commit_pair(&acc_full[0]);
                umma_commit_pair(&acc_full[1]);
            }
        }
    } else {
        const int quarter = warp & 3;
        OutT* y = (OutT*)p.y;
        uint32_t done = 0;
        bool ok = true;
        for (int tile = pair; tile < n_tiles && ok; tile += pairs, ++done) {
            const uint32_t b = done & 1;
            if (!mbar_wait(&acc_full[b], (done >> 1) & 1)) { if (lane == 0) *failed = 3; ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int r = (tile % tiles_m) * 256 + 128 * (int)rank + 32 * quarter + lane;   // activation row
            const int n0 = (tile / tiles_m) * PAIR_BN;
#pragma unroll 1
            for (int c0 = 0; c0 < PAIR_BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(32 * quarter) << 16) + 256 * b + (uint32_t)c0, v);
                const int n = n0 + c0;
                if (r >= p.R || n >= p.N) continue;
                float o[32];
                if (p.epilogue == GEMM_EPI_GEGLU) {
                    // weight rows come as 8 gates then their 8 ups: 32 columns make 16 outputs
#pragma unroll
                    for (int g = 0; g < 2; ++g)
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            o[8 * g + i] = gemm_gelu_tanh(__uint_as_float(v[16 * g + i])) *
                                           __uint_as_float(v[16 * g + 8 + i]);
                    OutT* dst = y + (size_t)r * p.y_stride + n / 2;
                    const int count = min(32, p.N - n) / 2;
                    if (count == 16 && ((uintptr_t)dst & 15) == 0 && sizeof(OutT) == 2) {
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            uint32_t w[4];
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const __nv_bfloat162 t2 = __floats2bfloat162_rn(o[8 * q + 2 * k], o[8 * q + 2 * k + 1]);
                                w[k] = *reinterpret_cast<const uint32_t*>(&t2);
                            }
                            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(dst) + 8 * q) =
                                make_uint4(w[0], w[1], w[2], w[3]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < count) dst[j] = from_f32<OutT>(o[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        o[j] = __uint_as_float(v[j]);
                        if (p.epilogue == GEMM_EPI_SOFTCAP) o[j] = p.cap * tanhf(o[j] / p.cap);
                    }
                    store_run<OutT>(y + (size_t)r * p.y_stride + n, o, min(32, p.N - n));
                }
            }
            // this warp has read its part of the accumulator
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_first_block(&acc_empty[b]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();          // the other block no longer touches this block's memory or barriers
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(512)
                     : "memory");
    }
    if (threadIdx.x == 0 && *failed) atomicExch(p.error_flag, *failed);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiled encode_fn() {
    static EncodeTiled fn = nullptr;
    if (fn) return fn;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = (EncodeTiled)ptr;
    return fn;
}

// A [rows, K] bfloat16 matrix with `stride` elements between rows, cut into boxes of
// box_rows x 64 elements, 128-byte swizzle, zeros outside.
static int make_map(CUtensorMap* map, const void* base, int rows, int K, long long stride,
                    int box_rows) {
    EncodeTiled enc = encode_fn();
    if (!enc) {
        sib_set_error("gemm_tcgen05: cuTensorMapEncodeTiled is not available");
        return -1;
    }
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)stride * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                     box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        sib_set_error("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d", (int)r);
        return -1;
    }
    return 0;
}

template <int BN, int STAGES, typename OutT>
static int launch_gemm(const CUtensorMap& mw, const CUtensorMap& mx, const GemmArgs& p,
                       cudaStream_t s) {
    const size_t smem = 1024 + (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + (2 * STAGES + 1) * 8 + 16;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, OutT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
        sib_set_error("gemm_tcgen05: shared memory: %s", cudaGetErrorString(e));
        return (int)e;
    }
    dim3 grid((p.N + BM - 1) / BM, (p.R + BN - 1) / BN);
    kernel<<<grid, 192, smem, s>>>(mw, mx, p);
    return sib_check_launch("gemm_tcgen05");
}

template <typename OutT>
static int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const GemmArgs& p, int sm_count,
                       cudaStream_t s) {
    const size_t smem = 1024 + (size_t)PAIR_STAGES * (128 * BK * 2 + (PAIR_BN / 2) * BK * 2) +
                        (2 * PAIR_STAGES + 4) * 8 + 16;
    auto kernel = gemm_tcgen05_pair_kernel<OutT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
        sib_set_error("gemm_tcgen05: shared memory: %s", cudaGetErrorString(e));
        return (int)e;
    }
    const int n_tiles = ((p.R + 255) / 256) * ((p.N + PAIR_BN - 1) / PAIR_BN);
    const int pairs = n_tiles < sm_count / 2 ? n_tiles : sm_count / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs, 1, 1);
    cfg.blockDim = dim3(192, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kernel, mx, mw, p);
    if (e != cudaSuccess) {
        sib_set_error("gemm_tcgen05: launch of the paired kernel failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return sib_check_launch("gemm_tcgen05");
}

static int g_sm_count[64] = {};

SIB_EXPORT int sib_gemm_tcgen05_supports(int R, int N, int K, long long x_stride) {
    return R > 0 && N > 0 && K > 0 && K % 8 == 0 && x_stride % 8 == 0;
}

// variant 0: the kernel that suits the number of rows; 1: always the one-block kernel.
static int gemm_tcgen05(const void* W, const void* x, void* y, int out_dtype, int R, int N, int K,
                        long long x_stride, int y_stride, int epilogue, float cap, int variant,
                        void* stream) {
    if (R == 0) return 0;
    SIB_REQUIRE(sib_gemm_tcgen05_supports(R, N, K, x_stride),
                "gemm_tcgen05: R=%d N=%d K=%d x_stride=%lld; K and the row stride must be multiples "
                "of 8", R, N, K, x_stride);
    SIB_REQUIRE(((uintptr_t)W % 16) == 0 && ((uintptr_t)x % 16) == 0,
                "gemm_tcgen05: operands must be 16-byte aligned");
    SIB_REQUIRE(epilogue != GEMM_EPI_GEGLU || N % 16 == 0,
                "gemm_tcgen05: the gated epilogue needs N (%d) in whole groups of 16", N);
    SIB_REQUIRE(epilogue != GEMM_EPI_SOFTCAP || cap > 0.f, "gemm_tcgen05: soft cap must be positive");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    SIB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, "gemm_tcgen05: no current device");
    int* error_flag = sib_error_word(SIB_ERR_GEMM_TCGEN05);   // the bounded waits' verdict
    if (!error_flag) return -1;
    if (!g_sm_count[dev]) {
        e = cudaDeviceGetAttribute(&g_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        SIB_REQUIRE(e == cudaSuccess && g_sm_count[dev] >= 2, "gemm_tcgen05: %s", cudaGetErrorString(e));
    }
    CUtensorMap mw, mx;
    if (R > 128 && variant != 1) {
        // many rows: tiles of 256 x 256 on pairs of SMs
        if (make_map(&mx, x, R, K, x_stride, 128)) return -1;
        if (make_map(&mw, W, N, K, K, PAIR_BN / 2)) return -1;
        GemmArgs pp{y, error_flag, R, N, K, y_stride, epilogue, cap};
        if (out_dtype == SIB_BF16)
            return launch_pair<__nv_bfloat16>(mx, mw, pp, g_sm_count[dev], (cudaStream_t)stream);
        if (out_dtype == SIB_F32)
            return launch_pair<float>(mx, mw, pp, g_sm_count[dev], (cudaStream_t)stream);
        SIB_REQUIRE(false, "gemm_tcgen05: unknown output type %d", out_dtype);
    }
    const int bn = R <= 32 ? 32 : R <= 64 ? 64 : R <= 128 ? 128 : 256;
    if (make_map(&mw, W, N, K, K, BM)) return -1;
    if (make_map(&mx, x, R, K, x_stride, bn)) return -1;
    GemmArgs p{y, error_flag, R, N, K, y_stride, epilogue, cap};
    cudaStream_t s = (cudaStream_t)stream;
#define GO(BN, ST)                                                              \
    do {                                                                        \
        if (out_dtype == SIB_BF16) return launch_gemm<BN, ST, __nv_bfloat16>(mw, mx, p, s); \
        if (out_dtype == SIB_F32) return launch_gemm<BN, ST, float>(mw, mx, p, s);          \
    } while (0)
    if (bn == 32) GO(32, 8);
    if (bn == 64) GO(64, 8);
    if (bn == 128) GO(128, 6);
    if (bn == 256) GO(256, 4);
#undef GO
    SIB_REQUIRE(false, "gemm_tcgen05: unknown output type %d", out_dtype);
}

SIB_EXPORT int sib_gemm_tcgen05(const void* W, const void* x, void* y, int out_dtype, int R, int N,
                                int K, long long x_stride, int y_stride, int epilogue, float cap,
                                void* stream) {
    return gemm_tcgen05(W, x, y, out_dtype, R, N, K, x_stride, y_stride, epilogue, cap, 0, stream);
}

// The one-block kernel whatever the number of rows (for comparison and tests).
SIB_EXPORT int sib_gemm_tcgen05_one_block(const void* W, const void* x, void* y, int out_dtype, int R,
                                          int N, int K, long long x_stride, int y_stride,
                                          int epilogue, float cap, void* stream) {
    return gemm_tcgen05(W, x, y, out_dtype, R, N, K, x_stride, y_stride, epilogue, cap, 1, stream);
}
