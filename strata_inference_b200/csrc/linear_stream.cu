// y[R, N] = x[R, K] . W[N, K]^T for at most 16 rows of bfloat16 activations: the
// weight-streaming product of decoding with the weights staged through shared memory.
//
// A block owns 128 weight rows (8 warps x 16) and a run of k.  One thread of a ninth
// warp feeds a ring of `stages` tiles of 128 rows x 64 k (16 KB each) with TMA loads
// (cp.async.bulk.tensor over a map of this GPU's own memory, 128-byte swizzle, no
// multicast), each completing on the tile's own barrier; the eight warps take the tiles
// in turn: 16-byte shared-memory loads whose swizzle makes them conflict-free, then
// mma.m16n8k16 with the weight rows as the A operand and the activation rows as B.
// Which k a fragment register stands for is permuted in the same way on both operands
// (a lane holds 16 consecutive k of its rows), so the sums are those of the plain
// product.
//
// The weights do not depend on the kernel that ran before, the activations do.  The
// launch is chained (programmatic dependent launch): a block starts while its
// predecessor still runs, its loader fills the whole ring at once, and only then do
// the eight warps wait for the predecessor (griddepcontrol.wait), fetch the block's
// activations into shared memory and start.  What is on the critical path after the
// predecessor's last write is one round trip for the activations and the arithmetic;
// the memory system has been busy with this kernel's weights all along.  Products with
// few weight rows split k over the blocks of a cluster (so that every SM streams);
// the partial sums meet in the first block's shared memory and are added in block
// order.  Epilogues: none, soft cap, gated tanh-GELU over rows that come as 8 gate rows
// followed by their 8 up rows.
//
// Every wait on a barrier is bounded; a wait that runs out leaves a code in the
// device's error word for this kernel (the host reports it) and the block winds down.
// Plain counterpart: tests/plain_gemma2.py (x @ W.T), gelu_tanh(), lm_head().
// Reference: src/model/layer.rs:22-43 (x . W^T, weights [out, in]).
#include <stdlib.h>

#include "common.cuh"
#include "tma.cuh"

namespace {

enum { LS_NONE = 0, LS_SOFTCAP = 1, LS_GEGLU = 2 };

constexpr int LS_BN = 128;                    // weight rows per block
constexpr int LS_BK = 64;                     // k per tile: one 128-byte swizzle row
constexpr int LS_STAGE = LS_BN * LS_BK * 2;   // bytes per tile
constexpr int LS_WARPS = 8;                   // consumer warps
constexpr int LS_THREADS = 32 * (LS_WARPS + 1);

struct StreamArgs {
    const __nv_bfloat16* x;
    void* y;
    int* error_flag;
    int R, N, K, x_stride, y_stride;
    float cap;
    int ks, stages;
};

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};\n" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
                 "r"(v.w)
                 : "memory");
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// Store into the same shared-memory offset of the cluster's block `rank`.
__device__ __forceinline__ void st_cluster_f4(uint32_t local_addr, uint32_t rank, float4 v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(remote) : "r"(local_addr), "r"(rank));
    asm volatile("st.shared::cluster.v4.f32 [%0], {%1,%2,%3,%4};\n" ::"r"(remote), "f"(v.x), "f"(v.y),
                 "f"(v.z), "f"(v.w)
                 : "memory");
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ls_gelu_tanh(float g) {
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
}

// NT: activation rows in tiles of 8 (1 or 2).
template <int NT, typename OutT, int EPI>
__global__ void __launch_bounds__(LS_THREADS, 1)
linear_stream_kernel(const __grid_constant__ CUtensorMap wmap, const StreamArgs p) {
    extern __shared__ uint8_t ls_raw[];
    const uint32_t raw = sib_smem_u32(ls_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;       // the swizzle wants 1024-byte tiles
    uint8_t* basep = ls_raw + (base - raw);
    const int stages = p.stages, ks = p.ks;
    const int KT = (p.K + LS_BK - 1) / LS_BK;
    const int kt_per = (KT + ks - 1) / ks;
    constexpr int ROWS = NT * 8;
    // ring of weight tiles | this block's activations [k tile][row][64] | partial sums of the
    // cluster's other blocks (first block only) | barriers
    const uint32_t ring = base;
    const uint32_t xres = ring + stages * LS_STAGE;
    const uint32_t peers = xres + kt_per * ROWS * 128;
    uint8_t* after = basep + stages * LS_STAGE + kt_per * ROWS * 128 + (ks - 1) * NT * 256 * 16;
    uint64_t* full = reinterpret_cast<uint64_t*>(after);
    uint64_t* empty = full + stages;
    volatile int* failed = reinterpret_cast<volatile int*>(empty + stages);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = blockIdx.y;
    const int n0 = blockIdx.x * LS_BN;
    const int kt0 = (int)((long long)rank * KT / ks);
    const int n_my = (int)((long long)(rank + 1) * KT / ks) - kt0;

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            sib_mbar_init(&full[s], 1);
            sib_mbar_init(&empty[s], LS_WARPS);
        }
        *failed = 0;
        sib_mbar_init_fence();
    }
    __syncthreads();
    if (ks > 1) cluster_arrive();      // matched by the wait before the partial sums travel

    float acc[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;

    if (warp == LS_WARPS) {
        // the loader: nothing it reads depends on the kernel before this one
        if (lane == 0) {
            for (int i = 0; i < n_my; ++i) {
                const int s = i % stages;
                if (i >= stages && !sib_mbar_wait(&empty[s], ((i / stages) - 1) & 1)) {
                    *failed = 1;
                    break;
                }
                sib_mbar_arrive_expect_tx(&full[s], LS_STAGE);
                sib_tma_load_2d(basep + s * LS_STAGE, &wmap, &full[s], (kt0 + i) * LS_BK, n0);
            }
        }
        __syncwarp();
    } else {
        pdl_wait();
        // this block's activations: rows of 128 bytes per (k tile, row), 16-byte chunk c of
        // row r kept at chunk c ^ (r % 8), as the TMA swizzle keeps the weights
        const int g = lane >> 2, t = lane & 3;
        const uint4 zero = make_uint4(0, 0, 0, 0);
        for (int idx = threadIdx.x; idx < n_my * ROWS * 8; idx += 32 * LS_WARPS) {
            const int c = idx & 7, r = (idx >> 3) % ROWS, kt = (idx >> 3) / ROWS;
            const int k = (kt0 + kt) * LS_BK + c * 8;
            uint4 v = zero;
            if (r < p.R && k < p.K)        // K is a multiple of 8: a chunk is inside or outside
                v = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)r * p.x_stride + k));
            sts128(xres + (kt * ROWS + r) * 128 + ((c ^ (r & 7)) << 4), v);
        }
        asm volatile("bar.sync 1, %0;\n" ::"n"(32 * LS_WARPS) : "memory");

        const uint32_t c0 = (uint32_t)((2 * t) ^ g) << 4, c1 = (uint32_t)((2 * t + 1) ^ g) << 4;
        const uint32_t wrow = (uint32_t)(16 * warp + g) * 128;
        for (int i = 0; i < n_my; ++i) {
            const int s = i % stages;
            if (!sib_mbar_wait(&full[s], (i / stages) & 1)) {
                *failed = 2;
                break;
            }
            const uint32_t tile = ring + s * LS_STAGE + wrow;
            const uint4 wa0 = lds128(tile + c0), wa1 = lds128(tile + c1);
            const uint4 wb0 = lds128(tile + 8 * 128 + c0), wb1 = lds128(tile + 8 * 128 + c1);
            __syncwarp();
            if (lane == 0) sib_mbar_arrive(&empty[s]);       // the tile is in registers
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const uint32_t xr = xres + (i * ROWS + 8 * j + g) * 128;
                const uint4 x0 = lds128(xr + c0), x1 = lds128(xr + c1);
                mma_16816(acc[j], wa0.x, wb0.x, wa0.y, wb0.y, x0.x, x0.y);
                mma_16816(acc[j], wa0.z, wb0.z, wa0.w, wb0.w, x0.z, x0.w);
                mma_16816(acc[j], wa1.x, wb1.x, wa1.y, wb1.y, x1.x, x1.y);
                mma_16816(acc[j], wa1.z, wb1.z, wa1.w, wb1.w, x1.z, x1.w);
            }
        }
        __syncwarp();
    }

    if (ks > 1) {
        cluster_wait();                // every block of the cluster is running
        if (rank > 0 && warp < LS_WARPS) {
#pragma unroll
            for (int j = 0; j < NT; ++j)
                st_cluster_f4(peers + (((rank - 1) * NT + j) * 256 + threadIdx.x) * 16, 0,
                              make_float4(acc[j][0], acc[j][1], acc[j][2], acc[j][3]));
        }
        cluster_arrive();
        cluster_wait();                // the partial sums have landed in the first block
    }
    __syncthreads();
    if (*failed) {
        if (threadIdx.x == 0) atomicExch(p.error_flag, *failed);
        return;
    }
    if (rank > 0 || warp == LS_WARPS) return;

    for (int b = 1; b < ks; ++b) {     // in block order
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const uint4 raw4 = lds128(peers + (((b - 1) * NT + j) * 256 + threadIdx.x) * 16);
            acc[j][0] += __uint_as_float(raw4.x);
            acc[j][1] += __uint_as_float(raw4.y);
            acc[j][2] += __uint_as_float(raw4.z);
            acc[j][3] += __uint_as_float(raw4.w);
        }
    }
    // acc[j][0], [1]: weight row na, activation rows r0, r0 + 1; [2], [3]: weight row na + 8
    OutT* y = reinterpret_cast<OutT*>(p.y);
    const int g = lane >> 2, t = lane & 3;
    const int na = n0 + 16 * warp + g;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int r0 = 8 * j + 2 * t;
        if (EPI == LS_GEGLU) {
            // rows g (gate) and g + 8 (up) of a 16-row group make output column n_out
            const int n_out = (n0 + 16 * warp) / 2 + g;
            if (na + 8 < p.N) {
                if (r0 < p.R)
                    y[(size_t)r0 * p.y_stride + n_out] =
                        from_f32<OutT>(ls_gelu_tanh(acc[j][0]) * acc[j][2]);
                if (r0 + 1 < p.R)
                    y[(size_t)(r0 + 1) * p.y_stride + n_out] =
                        from_f32<OutT>(ls_gelu_tanh(acc[j][1]) * acc[j][3]);
            }
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float o = acc[j][c];
                if (EPI == LS_SOFTCAP) o = p.cap * tanhf(o / p.cap);
                const int n = na + (c >= 2 ? 8 : 0), r = r0 + (c & 1);
                if (n < p.N && r < p.R) y[(size_t)r * p.y_stride + n] = from_f32<OutT>(o);
            }
        }
    }
}

int g_ls_sm_count[64] = {};

size_t stream_smem(int NT, int KT, int ks, int stages) {
    const int kt_per = (KT + ks - 1) / ks;
    return 1024 + (size_t)stages * LS_STAGE + (size_t)kt_per * NT * 8 * 128 +
           (size_t)(ks - 1) * NT * 256 * 16 + (size_t)2 * stages * 8 + 16;
}

template <int NT, typename OutT, int EPI>
int launch_stream(const CUtensorMap& wmap, const StreamArgs& p, size_t smem, cudaStream_t s) {
    auto kernel = linear_stream_kernel<NT, OutT, EPI>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
        sib_set_error("linear_stream: shared memory (%zu bytes): %s", smem, cudaGetErrorString(e));
        return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.N + LS_BN - 1) / LS_BN, p.ks, 1);
    cfg.blockDim = dim3(LS_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = p.ks;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sib_chained_launches() ? 2 : 1;
    sib_same_carveout(kernel);
    e = cudaLaunchKernelEx(&cfg, kernel, wmap, p);
    if (e != cudaSuccess) {
        sib_set_error("linear_stream: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return sib_check_launch("linear_stream");
}

// How many blocks of a cluster share a tile of weight rows: the split that fills the SMs
// best, each block keeping at least two tiles of k.
int choose_ksplit(int tiles, int KT, int sms) {
    if (tiles >= sms) return 1;
    int best = 1;
    double best_fill = 0.0;
    for (int ks = 1; ks <= 8 && KT / ks >= 2; ++ks) {
        const int units = tiles * ks;
        const int waves = (units + sms - 1) / sms;
        const double fill = (double)units / ((double)waves * sms);
        if (fill > best_fill + 0.02) {
            best_fill = fill;
            best = ks;
        }
    }
    return best;
}

}  // namespace

SIB_EXPORT int sib_linear_stream_supports(int R, int N, int K, int x_stride) {
    return R > 0 && R <= 16 && N > 0 && K > 0 && K % 8 == 0 && x_stride % 8 == 0;
}

// ksplit, stages: 0 lets the launcher choose.
SIB_EXPORT int sib_linear_stream(const void* W, const void* x, void* y, int out_dtype, int R, int N,
                                 int K, int x_stride, int y_stride, int epilogue, float cap,
                                 int ksplit, int stages, void* stream) {
    if (R == 0) return 0;
    SIB_REQUIRE(sib_linear_stream_supports(R, N, K, x_stride),
                "linear_stream: R=%d N=%d K=%d x_stride=%d; 1 to 16 rows, K and the row stride "
                "multiples of 8", R, N, K, x_stride);
    SIB_REQUIRE(((uintptr_t)W % 16) == 0 && ((uintptr_t)x % 16) == 0,
                "linear_stream: operands must be 16-byte aligned");
    SIB_REQUIRE(epilogue != LS_GEGLU || N % 16 == 0,
                "linear_stream: the gated epilogue needs N (%d) in whole groups of 16", N);
    SIB_REQUIRE(epilogue != LS_SOFTCAP || cap > 0.f, "linear_stream: soft cap must be positive");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    SIB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, "linear_stream: no current device");
    if (!g_ls_sm_count[dev]) {
        e = cudaDeviceGetAttribute(&g_ls_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        SIB_REQUIRE(e == cudaSuccess && g_ls_sm_count[dev] > 0, "linear_stream: %s",
                    cudaGetErrorString(e));
    }
    int* error_flag = sib_error_word(SIB_ERR_LINEAR_STREAM);
    if (!error_flag) return -1;
    const int NT = R <= 8 ? 1 : 2;
    const int KT = (K + LS_BK - 1) / LS_BK;
    const int tiles = (N + LS_BN - 1) / LS_BN;
    SIB_REQUIRE(ksplit >= 0 && ksplit <= 8 && stages >= 0 && stages <= 12,
                "linear_stream: ksplit %d (0 to 8) or stages %d (0 to 12)", ksplit, stages);
    int ks = ksplit > 0 ? ksplit : choose_ksplit(tiles, KT, g_ls_sm_count[dev]);
    if (ks > KT) ks = KT;
    // the block's activations must fit beside the ring: split k further if they do not
    while (stream_smem(NT, KT, ks, 2) > 200 * 1024 && ks < 8 && ks < KT) ++ks;
    const int kt_per = (KT + ks - 1) / ks;
    static int env_stages = -1, env_ks = -1;
    if (env_stages < 0) {
        const char* v = getenv("SIB_LS_STAGES");
        env_stages = v ? atoi(v) : 0;
        const char* k = getenv("SIB_LS_KSPLIT");
        env_ks = k ? atoi(k) : 0;
    }
    if (ksplit == 0 && env_ks > 0 && tiles < g_ls_sm_count[dev] / 2) {
        ks = env_ks > KT ? KT : env_ks;
    }
    int st = stages > 0 ? stages : (env_stages > 0 ? env_stages : 6);
    if (st > kt_per) st = kt_per;
    while (st > 2 && stream_smem(NT, KT, ks, st) > 200 * 1024) --st;
    const size_t smem = stream_smem(NT, KT, ks, st);
    SIB_REQUIRE(smem <= 227 * 1024, "linear_stream: K=%d needs %zu bytes of shared memory a block",
                K, smem);
    CUtensorMap wmap;
    if (sib_make_bf16_map(&wmap, W, N, K, K, LS_BN, "linear_stream")) return -1;
    StreamArgs p{(const __nv_bfloat16*)x, y, error_flag, R, N, K, x_stride, y_stride, cap, ks, st};
    cudaStream_t s = (cudaStream_t)stream;
#define GO(NTV, OUT, EPI) return launch_stream<NTV, OUT, EPI>(wmap, p, smem, s)
#define BY_EPI(NTV, OUT)                                \
    do {                                                \
        if (epilogue == LS_NONE) GO(NTV, OUT, LS_NONE); \
        if (epilogue == LS_SOFTCAP) GO(NTV, OUT, LS_SOFTCAP); \
        if (epilogue == LS_GEGLU) GO(NTV, OUT, LS_GEGLU); \
    } while (0)
    if (out_dtype == SIB_BF16) {
        if (NT == 1) BY_EPI(1, __nv_bfloat16);
        BY_EPI(2, __nv_bfloat16);
    } else if (out_dtype == SIB_F32) {
        if (NT == 1) BY_EPI(1, float);
        BY_EPI(2, float);
    }
#undef BY_EPI
#undef GO
    SIB_REQUIRE(false, "linear_stream: unknown output type %d or epilogue %d", out_dtype, epilogue);
}
