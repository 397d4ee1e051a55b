// y[R, N] = x[R, K] . W[N, K]^T for some rows (R <= 128), bfloat16 operands, 32-bit
// accumulation, on the fifth-generation tensor cores: the weight-streaming product of
// steps with more rows than linear_skinny.cu takes and fewer than fill a library product's
// tiles (decoding at batch 17 to 128, short prompts).  Every weight is read once; the time
// is the time to read it.  The engine uses it for products with very many weight rows (the
// logits); for a layer's own matrices the library product is as fast or faster (see the
// launcher's notes at the end of this file).
//
// The operands are swapped against the usual product: a block's 128 weight rows are the M
// side of tcgen05.mma (operand A, K-major in shared memory), the step's rows, rounded up to
// a multiple of 16, the N side (operand B), and the accumulator [128 weight rows x rows]
// lies in tensor memory.  A ring of TMA stages (64 of k: 16 KB of weights and the rows' 128
// bytes each) feeds one thread that issues the MMAs; the weights of the first stages are
// asked for before the kernel ahead of this one has finished, the rows after it.
//
//   warp 0      TMA: weight tiles (two boxes of 64 rows) and row tiles into the ring
//   warp 1      allocates tensor memory; one lane issues the MMAs and frees the stages
//   warps 2-5   epilogue: accumulator -> shared memory of the block that owns the weight
//               row -> sum over the blocks that split k -> epilogue -> y
//
// Few weight rows: `ksplit` blocks (a cluster) share a tile of weight rows and split k.
// Each writes its partial sums into the shared memory of the block that owns the weight row
// (128 / ksplit consecutive rows each), and the owners add the parts in block order.
//
// Epilogues: none; soft cap (cap * tanh(y / cap)); gated tanh-GELU, for which the weight
// rows come in groups of 16 (8 gate rows, then the 8 matching up rows) and y gets N / 2
// columns.  Every wait is bounded; a wait that runs out sets the kernel's error word.
//
// Plain counterpart: tests/plain_gemma2.py (x @ W.T), gelu_tanh(), lm_head().
// Reference: src/model/layer.rs:22-43 (x . W^T, weights [out, in]).
#include <cuda.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "tma.cuh"

namespace {

constexpr int TILE_N = 128;      // weight rows per block: the M of the MMA
constexpr int BK = 64;           // k per stage: 128 bytes of a row
constexpr int MAX_STAGES = 8;
constexpr uint32_t A_BYTES = TILE_N * 128;
enum { EPI_NONE = 0, EPI_SOFTCAP = 1, EPI_GEGLU = 2 };

struct RowsArgs {
    void* y;
    int* error_flag;
    int R, Rp, N, K, y_stride;
    int ksplit, stages, tmem_cols;
    float cap;
};

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;\n" ::"r"(sib_smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// K-major operand tile: rows of 128 bytes (64 elements of k), 8-row groups 1024 bytes
// apart, 128-byte swizzle.
__device__ __forceinline__ uint64_t desc_k_major(uint32_t tile_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((tile_addr >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
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
// arrives on `bar` once the MMAs issued so far have run
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                     sib_smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// the shared::cluster address of this block's shared address `a` in block `rank` of the cluster
__device__ __forceinline__ uint32_t in_block(uint32_t a, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(a), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ float gelu_tanh_f(float g) {
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
}

template <int EPI, typename OutT>
__global__ void __launch_bounds__(192)
linear_rows_tc_kernel(const __grid_constant__ CUtensorMap wmap,
                      const __grid_constant__ CUtensorMap xmap, RowsArgs p) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t b_bytes = (uint32_t)p.Rp * 128;
    const uint32_t stage_bytes = A_BYTES + b_bytes;
    unsigned char* ring = base;
    // parts of the blocks that split k: [ksplit][128 / ksplit rows][Rp + 4] (none without a split)
    float* red = reinterpret_cast<float*>(ring + (size_t)p.stages * stage_bytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(red + (p.ksplit > 1 ? (size_t)TILE_N * (p.Rp + 4) : 0));
    uint64_t* empty = full + MAX_STAGES;
    uint64_t* acc_full = empty + MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    int* failed = reinterpret_cast<int*>(tmem_slot + 1);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ksplit = p.ksplit, stages = p.stages;
    const int rank = ksplit > 1 ? (int)cluster_rank() : 0;
    const int tile = blockIdx.x;
    // this block's run of 64-wide steps of k
    const int total_steps = (p.K + BK - 1) / BK;
    const int per = total_steps / ksplit, rem = total_steps % ksplit;
    const int k_begin = rank * per + min(rank, rem);
    const int n_steps = per + (rank < rem ? 1 : 0);

    const int n0 = tile * TILE_N;
    auto load_a = [&](int i) {
        unsigned char* a = ring + (size_t)(i % stages) * stage_bytes;
        sib_tma_load_2d(a, &wmap, &full[i % stages], (k_begin + i) * BK, n0);
        sib_tma_load_2d(a + A_BYTES / 2, &wmap, &full[i % stages], (k_begin + i) * BK, n0 + 64);
    };
    const int pre = min(stages, n_steps);
    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&wmap) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(&xmap) : "memory");
        for (int s = 0; s < stages; ++s) {
            sib_mbar_init(&full[s], 1);
            sib_mbar_init(&empty[s], 1);
        }
        sib_mbar_init(acc_full, 1);
        *failed = 0;
        sib_mbar_init_fence();
        // The weights do not depend on the kernel before this one: the first stages'
        // weights are on their way before anything else of this block is set up, while
        // that kernel may still be running.
        for (int i = 0; i < pre; ++i) {
            mbar_expect_tx(&full[i], A_BYTES);
            load_a(i);
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                         sib_smem_u32(tmem_slot)),
                     "r"((uint32_t)p.tmem_cols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    // (the blocks of a cluster write into each other's shared memory at the end: each says
    // here that it is running, and nobody writes before all have said so)
    if (ksplit > 1) cluster_arrive();

    if (warp == 0) {
        if (lane == 0) {
            auto load_b = [&](int i) {
                unsigned char* a = ring + (size_t)(i % stages) * stage_bytes;
                sib_tma_load_2d(a + A_BYTES, &xmap, &full[i % stages], (k_begin + i) * BK, 0);
            };
            // (the first stages' weights were asked for above; the rows need the kernel ahead)
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                sib_mbar_arrive_expect_tx(&full[i], b_bytes);
                load_b(i);
            }
            int issued = pre;
            for (int i = pre; i < n_steps; ++i) {
                const int s = i % stages;
                if (!sib_mbar_wait(&empty[s], ((i / stages) - 1) & 1)) {
                    *failed = 1;
                    break;
                }
                sib_mbar_arrive_expect_tx(&full[s], stage_bytes);
                load_a(i);
                load_b(i);
                issued = i + 1;
            }
            if (*failed) {
                // let no copy of this block be in flight when it ends
                for (int i = max(0, issued - stages); i < issued; ++i)
                    sib_mbar_wait(&full[i % stages], (i / stages) & 1);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // D[128 x Rp] (f32) += A[128 x 16] B[Rp x 16]^T, both K-major bfloat16
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) |
                                   ((uint32_t)(p.Rp >> 3) << 17) | ((uint32_t)(TILE_N >> 4) << 24);
            for (int i = 0; i < n_steps; ++i) {
                const int s = i % stages;
                if (*failed) break;
                if (!sib_mbar_wait(&full[s], (i / stages) & 1)) {
                    *failed = 2;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t a = sib_smem_u32(ring + (size_t)s * stage_bytes);
                const uint64_t da = desc_k_major(a), db = desc_k_major(a + A_BYTES);
#pragma unroll
                for (int j = 0; j < BK / 16; ++j)
                    umma_bf16(tmem, da + 2 * j, db + 2 * j, idesc, (i > 0 || j > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            umma_commit(acc_full);        // (also when a wait ran out: nobody waits for nothing)
        }
        __syncwarp();
    }

    const int rpo = TILE_N / ksplit;      // weight rows a block of the cluster owns
    const int pitch = p.Rp + 4;           // floats between the weight rows of a part
    OutT* y = reinterpret_cast<OutT*>(p.y);
    if (warp >= 2) {
        const int quarter = warp & 3;                  // the tensor-memory lanes this warp may read
        const int row = 32 * quarter + lane;           // weight row of the tile
        pdl_wait();                                    // (y may be memory the kernel ahead still reads)
        bool ok = sib_mbar_wait(acc_full, 0);
        if (!ok && lane == 0) *failed = 3;
        ok = __all_sync(0xffffffffu, ok && !*failed);     // (one answer per warp)
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        const uint32_t lane_addr = tmem + ((uint32_t)(32 * quarter) << 16);
        if (ksplit == 1) {
            // the whole sum is here: straight from tensor memory to y (a warp writes 32
            // neighbouring columns of a row of y at a time)
            const int n = tile * TILE_N + row;
            for (int c = 0; c < p.Rp && ok; c += 16) {
                uint32_t v[16];
                tmem_ld16(lane_addr + c, v);
                if (EPI == EPI_GEGLU) {
                    // rows j (gate) and j + 8 (up) of a group of 16 make column (group start) / 2 + j
                    const bool gate = (row & 8) == 0;
                    const int col = (tile * TILE_N + (row & ~15)) / 2 + (row & 7);
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float up = __shfl_down_sync(0xffffffffu, __uint_as_float(v[j]), 8);
                        if (gate && c + j < p.R && n + 8 < p.N)
                            y[(size_t)(c + j) * p.y_stride + col] =
                                from_f32<OutT>(gelu_tanh_f(__uint_as_float(v[j])) * up);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float s = __uint_as_float(v[j]);
                        if (EPI == EPI_SOFTCAP) s = p.cap * tanhf(s / p.cap);
                        if (c + j < p.R && n < p.N) y[(size_t)(c + j) * p.y_stride + n] = from_f32<OutT>(s);
                    }
                }
            }
        } else {
            // this block's part of weight row `row`, 16 bytes at a time, into the shared
            // memory of the block that owns the row: red[part][row of the owner][rows]
            cluster_wait();
            const int owner = row / rpo, local = row % rpo;
            const uint32_t dst = in_block(sib_smem_u32(red), (uint32_t)owner) +
                                 (uint32_t)(((size_t)rank * rpo + local) * pitch * sizeof(float));
            for (int c = 0; c < p.Rp; c += 16) {
                uint32_t v[16];
                if (ok) {
                    tmem_ld16(lane_addr + c, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; j += 4)
                    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};\n" ::"r"(
                                     dst + (uint32_t)(c + j) * 4u),
                                 "r"(v[j]), "r"(v[j + 1]), "r"(v[j + 2]), "r"(v[j + 3])
                                 : "memory");
            }
        }
    } else if (ksplit > 1) {
        cluster_wait();
    }
    if (ksplit > 1) {
        // every part is in its owner's shared memory
        cluster_arrive();
        cluster_wait();
        if (warp >= 2 && !*failed) {
            const int te = threadIdx.x - 64;               // 0..127
            const int n_first = tile * TILE_N + rank * rpo;
            auto total = [&](int r, int local) {
                float s = 0.f;
                for (int b = 0; b < ksplit; ++b)           // in block order
                    s += red[((size_t)b * rpo + local) * pitch + r];
                return s;
            };
            if (EPI == EPI_GEGLU) {
                const int half = rpo / 2;
                for (int idx = te; idx < half * p.R; idx += 128) {
                    const int o = idx % half, r = idx / half;
                    const int local = 16 * (o / 8) + (o % 8);
                    if (n_first + local + 8 < p.N)
                        y[(size_t)r * p.y_stride + (n_first / 2 + o)] =
                            from_f32<OutT>(gelu_tanh_f(total(r, local)) * total(r, local + 8));
                }
            } else {
                for (int idx = te; idx < rpo * p.R; idx += 128) {
                    const int local = idx % rpo, r = idx / rpo;
                    const int n = n_first + local;
                    if (n < p.N) {
                        float s = total(r, local);
                        if (EPI == EPI_SOFTCAP) s = p.cap * tanhf(s / p.cap);
                        y[(size_t)r * p.y_stride + n] = from_f32<OutT>(s);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem),
                     "r"((uint32_t)p.tmem_cols)
                     : "memory");
    }
    if (threadIdx.x == 0 && *failed) atomicExch(p.error_flag, *failed);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
int g_rows_tc_sms[64] = {};

int env_int(const char* name, int fallback) {
    const char* v = getenv(name);
    return v ? atoi(v) : fallback;
}

// Tensor maps of weight matrices, kept: a model's matrices stay where they are.
int weight_map(CUtensorMap* out, const void* W, int N, int K) {
    static std::mutex mutex;
    static std::map<std::tuple<const void*, int, int>, CUtensorMap> maps;
    std::lock_guard<std::mutex> guard(mutex);
    const auto key = std::make_tuple(W, N, K);
    auto it = maps.find(key);
    if (it == maps.end()) {
        CUtensorMap m;
        if (sib_make_bf16_map(&m, W, N, K, K, 64, "linear_rows_tc")) return -1;
        if (maps.size() > 4096) maps.clear();
        it = maps.emplace(key, m).first;
    }
    *out = it->second;
    return 0;
}

template <int EPI, typename OutT>
int launch_rows(const CUtensorMap& wmap, const CUtensorMap& xmap, const RowsArgs& p, size_t smem,
                int tiles, cudaStream_t s) {
    auto kernel = linear_rows_tc_kernel<EPI, OutT>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
        sib_set_error("linear_rows_tc: shared memory: %s", cudaGetErrorString(e));
        return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tiles, p.ksplit, 1);
    cfg.blockDim = dim3(192, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.ksplit;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sib_chained_launches() ? 2 : 1;
    e = cudaLaunchKernelEx(&cfg, kernel, wmap, xmap, p);
    if (e != cudaSuccess) {
        sib_set_error("linear_rows_tc: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return sib_check_launch("linear_rows_tc");
}

}  // namespace

// The most rows this product takes.
SIB_EXPORT int sib_linear_rows_tc_max_rows() { return 128; }

// `ksplit` (0: chosen) blocks share a tile of 128 weight rows; `stages` (0: chosen) ring slots.
//
// Measured alone (CUDA graph of 32 launches on weights larger than L2, Gemma2-2B shapes, one
// B200), this kernel / cuBLAS, in us:
//   rows   logits 256000x2304   gate|up 18432x2304 (+GeGLU here)   down 2304x9216   q|k|v 4096x2304   output 2304x2048
//    32        198 / 271*             19.2 / 19.7                    13.0 / 14.3       8.4 / 6.4         6.4 / 5.7
//    64        223 / 324*             23.5 / 22.1                    15.6 / 14.4      10.5 / 6.9         8.6 / 5.8
//   128        279 / 430*             29.2 / 24.7                    32.8 / 14.9      33.5 / 7.0        21.3 / 6.0
// (*: the one-block tcgen05 product of gemm_tcgen05.cu with the soft-cap epilogue, which the
// logits used before).  With many tiles (no split of k) it streams at 0.91 of the copy
// bandwidth; a layer's matrices have 18 to 144 tiles, so a launch is one or two waves whose
// start (tensor memory, barriers, the first tiles' latency) and end (accumulator out, the
// exchange between the blocks that split k) are not hidden by anything: about 5 us a launch.
// Inside a decode step (batch 24, Gemma2-2B shape) with every product of a layer on this
// kernel the step took 4.57 ms against 4.22 ms with the library's products.
SIB_EXPORT int sib_linear_rows_tc(const void* W, const void* x, void* y, int out_dtype, int R, int N,
                                  int K, int x_stride, int y_stride, int epilogue, float cap,
                                  int ksplit, int stages, void* stream) {
    if (R == 0) return 0;
    SIB_REQUIRE(R > 0 && R <= 128, "linear_rows_tc: %d rows; this product takes 1 to 128", R);
    SIB_REQUIRE(N > 0 && K > 0 && K % 8 == 0 && x_stride % 8 == 0 && x_stride >= K,
                "linear_rows_tc: N=%d K=%d x_stride=%d; K and the stride must be multiples of 8", N, K,
                x_stride);
    SIB_REQUIRE(((uintptr_t)W % 16) == 0 && ((uintptr_t)x % 16) == 0 && y != nullptr,
                "linear_rows_tc: operands must be 16-byte aligned");
    SIB_REQUIRE(epilogue != EPI_GEGLU || N % 16 == 0,
                "linear_rows_tc: the gated epilogue needs N (%d) in whole groups of 16", N);
    SIB_REQUIRE(epilogue != EPI_SOFTCAP || cap > 0.f, "linear_rows_tc: soft cap must be positive");
    SIB_REQUIRE(ksplit >= 0 && ksplit <= 8 && (ksplit & (ksplit - 1)) == 0 && stages >= 0 &&
                    stages <= MAX_STAGES,
                "linear_rows_tc: ksplit %d (0, 1, 2, 4 or 8) or stages %d (0 to %d)", ksplit, stages,
                MAX_STAGES);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    SIB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, "linear_rows_tc: no current device");
    if (!g_rows_tc_sms[dev]) {
        e = cudaDeviceGetAttribute(&g_rows_tc_sms[dev], cudaDevAttrMultiProcessorCount, dev);
        SIB_REQUIRE(e == cudaSuccess && g_rows_tc_sms[dev] > 0, "linear_rows_tc: %s", cudaGetErrorString(e));
    }
    const int sms = g_rows_tc_sms[dev];
    int* error_flag = sib_error_word(SIB_ERR_LINEAR_ROWS_TC);
    if (!error_flag) return -1;

    const int Rp = (R + 15) / 16 * 16;
    int tmem_cols = 32;
    while (tmem_cols < Rp) tmem_cols *= 2;
    const int tiles = (N + TILE_N - 1) / TILE_N;
    const int total_steps = (K + BK - 1) / BK;
    if (ksplit == 0) ksplit = env_int("SIB_ROWS_TC_KSPLIT", 0);
    if (ksplit == 0) {
        // as many blocks as two per SM hold, none with fewer than two steps of k
        ksplit = 1;
        while (ksplit < 8 && tiles * ksplit * 2 <= 2 * sms && total_steps >= 4 * ksplit) ksplit *= 2;
    }
    while (ksplit > 1 && total_steps < ksplit) ksplit /= 2;
    const size_t stage_bytes = A_BYTES + (size_t)Rp * 128;
    const size_t fixed = 1024 + (ksplit > 1 ? (size_t)TILE_N * (Rp + 4) * sizeof(float) : 0) +
                         (2 * MAX_STAGES + 1) * 8 + 16;
    if (stages == 0) stages = env_int("SIB_ROWS_TC_STAGES", 0);
    if (stages == 0) {
        if (ksplit == 1 && tiles >= 4 * sms) {
            // many waves of blocks: two stages each, so that as many blocks as possible share
            // an SM and one block's start and end lie under the others' streaming (measured
            // on the 256 000 x 2 304 logits product: 198-279 us for 17-128 rows with two
            // stages, 209-297 us with three or four, 286-394 us with six)
            stages = 2;
        } else {
            // two blocks per SM if each still gets three stages, else one block with what fits.
            // (Measured inside a decode step of 24 rows with every product on this kernel:
            // blocks of 98 KB, two of which fill an SM's shared memory, made the step 6.45 ms
            // with chained launches and 4.55 ms without; blocks of 78 KB 4.57 ms with them.
            // A kernel that takes all of an SM's shared memory does not get along with
            // programmatic dependent launches of its neighbours; so at most 80 KB a block.)
            const size_t two = 80 * 1024, one = 224 * 1024;
            stages = (int)((two - fixed) / stage_bytes);
            if (fixed > two || stages < 3) stages = (int)((one - fixed) / stage_bytes);
            if (stages > MAX_STAGES) stages = MAX_STAGES;
        }
    }
    const int steps_per_block = (total_steps + ksplit - 1) / ksplit;
    if (stages > steps_per_block) stages = steps_per_block;
    const size_t smem = fixed + stages * stage_bytes;
    SIB_REQUIRE(stages >= 1 && smem <= 227 * 1024, "linear_rows_tc: %d stages of %zu bytes do not fit",
                stages, stage_bytes);

    CUtensorMap wmap, xmap;
    if (weight_map(&wmap, W, N, K)) return -1;
    if (sib_make_bf16_map(&xmap, x, R, K, x_stride, Rp, "linear_rows_tc")) return -1;
    RowsArgs p{y, error_flag, R, Rp, N, K, y_stride, ksplit, stages, tmem_cols, cap};
    cudaStream_t s = (cudaStream_t)stream;
#define GO(EPI, OUT) return launch_rows<EPI, OUT>(wmap, xmap, p, smem, tiles, s)
    if (out_dtype == SIB_BF16) {
        if (epilogue == EPI_NONE) GO(EPI_NONE, __nv_bfloat16);
        if (epilogue == EPI_SOFTCAP) GO(EPI_SOFTCAP, __nv_bfloat16);
        if (epilogue == EPI_GEGLU) GO(EPI_GEGLU, __nv_bfloat16);
    } else if (out_dtype == SIB_F32) {
        if (epilogue == EPI_NONE) GO(EPI_NONE, float);
        if (epilogue == EPI_SOFTCAP) GO(EPI_SOFTCAP, float);
        if (epilogue == EPI_GEGLU) GO(EPI_GEGLU, float);
    }
#undef GO
    SIB_REQUIRE(false, "linear_rows_tc: unknown output type %d or epilogue %d", out_dtype, epilogue);
}
