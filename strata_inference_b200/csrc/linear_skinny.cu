// y[R, N] = x[R, K] . W[N, K]^T for a few rows (R <= 64), bfloat16 operands,
// 32-bit accumulation: the weight-streaming product of decoding, where every
// weight is read once and the time is the time to read it.
//
// The weight tile is the A operand of mma.m16n8k16 (16 weight rows), the
// activations are the B operand (8 activation rows per tile).  Fragments are
// loaded straight from global memory with 16-byte loads: lane (g, t) reads 16
// consecutive k of weight rows g and g + 8 and of activation row g.  Which k a
// fragment register stands for is permuted the same way on both operands, so
// the sums are those of the plain product.  The 8 warps of a block take
// alternating 64-wide blocks of k of the same 16 (or 32) weight rows; their
// partial sums are added in warp order through shared memory.
//
// The q|k|v product of attention can rotate q and k and write k and v into the paged
// cache itself (RopeTail): a tile then takes 8 weight rows of a head's first half and
// the 8 rows that produce their rotation partners (half a head further on), so that
// both elements of a pair end up in one thread; no weight is moved for it, only the
// two row pointers of a tile change.  Rotation and cache layout are those of
// rope_cache.cu.
//
// Epilogues: none; soft cap (cap * tanh(y / cap)); gated tanh-GELU, for which
// the weight rows come in groups of 16: 8 gate rows, then the 8 matching up
// rows, and y gets N / 2 columns.
// Plain counterpart: tests/plain_gemma2.py (x @ W.T), gelu_tanh(), lm_head().
// Reference: src/model/layer.rs:22-43 (x . W^T, weights [out, in]).
#include <cooperative_groups.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"

namespace cg = cooperative_groups;

enum { EPI_NONE = 0, EPI_SOFTCAP = 1, EPI_GEGLU = 2, EPI_ROPE = 3 };

// What the q|k|v product needs to rotate and store (see rope_cache.cu for the cache layout).
struct RopeTail {
    const int* row_pos;        // [rows] absolute position
    const int* row_seq;        // [rows] index into the step's sequences
    const int* seq_slot;       // [seqs]
    const int* seq_end;        // [seqs] length after this step
    const float* inv_freq;     // [head_dim / 2]
    __nv_bfloat16* k_pool;     // null: q only, nothing is stored
    __nv_bfloat16* v_pool;
    const int* page_table;     // [slots, max_pages]
    int n_heads, n_kv, head_dim;
    int max_pages, page_tokens, ring_tokens;
};

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld16(const __nv_bfloat16* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
// Weights are read once: keep them out of L1.
__device__ __forceinline__ uint4 ld16_stream(const __nv_bfloat16* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}

__device__ __forceinline__ float gelu_tanh_f(float g) {
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
}

// NT: activation tiles of 8 rows; MT: weight tiles of 16 rows per block.
template <int NT, int MT, typename OutT, int EPI>
__device__ __forceinline__ void skinny_linear_body(
    const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x, OutT* __restrict__ y,
    int R, int N, int K, int x_stride, int y_stride, float cap, int ksplit, const RopeTail& rope) {
    // [8 warps][MT][NT][32 lanes][4], then [ksplit - 1][MT][NT][32][4] for the other
    // blocks of the cluster (used in the cluster's first block only)
    extern __shared__ float red[];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = ksplit > 1 ? (int)cluster.block_rank() : 0;
    // Every block of the cluster must be running before its memory is written.  The blocks
    // say so here and look for the others' word only when they have their sums: the meeting
    // costs the loads below nothing.
    if (ksplit > 1) asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory");
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * (16 * MT);
    // the tile's two runs of 8 weight rows: consecutive, or (q and k heads of the rotating
    // product) half a head apart
    int run_a = n0, run_b = n0 + 8;
    if (EPI == EPI_ROPE) {
        const int per_head = rope.head_dim / 16;
        const int head = blockIdx.x / per_head, i = blockIdx.x % per_head;
        if (head < rope.n_heads + rope.n_kv) {
            run_a = head * rope.head_dim + 8 * i;
            run_b = run_a + rope.head_dim / 2;
        }
    }

    float acc[MT][NT][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < NT; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[m][j][c] = 0.f;

    const __nv_bfloat16* wrow[MT][2];
#pragma unroll
    for (int m = 0; m < MT; ++m) {
        wrow[m][0] = W + (size_t)min(run_a + 16 * m + g, N - 1) * K;
        wrow[m][1] = W + (size_t)min(run_b + 16 * m + g, N - 1) * K;
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);

    // The weights do not depend on the kernel before this one: pull this warp's part
    // of them towards L2 while that kernel is still running, then wait for it.
    pdl_trigger();
    if (t == 0) {
        for (int kb = (rank * 8 + warp) * 64; kb < K; kb += ksplit * 8 * 64) {
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wrow[m][0] + kb));
                asm volatile("prefetch.global.L2 [%0];\n" ::"l"(wrow[m][1] + kb));
            }
        }
    }
    pdl_wait();

#pragma unroll 2
    for (int kb = (rank * 8 + warp) * 64; kb < K; kb += ksplit * 8 * 64) {
        const int k = kb + 16 * t;
        const bool v0 = k + 8 <= K, v1 = k + 16 <= K;  // K is a multiple of 8
        uint4 wa[MT][2], wb[MT][2];
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            wa[m][0] = v0 ? ld16_stream(wrow[m][0] + k) : zero;
            wa[m][1] = v1 ? ld16_stream(wrow[m][0] + k + 8) : zero;
            wb[m][0] = v0 ? ld16_stream(wrow[m][1] + k) : zero;
            wb[m][1] = v1 ? ld16_stream(wrow[m][1] + k + 8) : zero;
        }
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const int r = 8 * j + g;
            uint4 x0 = zero, x1 = zero;
            if (r < R) {
                const __nv_bfloat16* xp = x + (size_t)r * x_stride + k;
                if (v0) x0 = ld16(xp);
                if (v1) x1 = ld16(xp + 8);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                mma_bf16_16816(acc[m][j], wa[m][0].x, wb[m][0].x, wa[m][0].y, wb[m][0].y, x0.x, x0.y);
                mma_bf16_16816(acc[m][j], wa[m][0].z, wb[m][0].z, wa[m][0].w, wb[m][0].w, x0.z, x0.w);
                mma_bf16_16816(acc[m][j], wa[m][1].x, wb[m][1].x, wa[m][1].y, wb[m][1].y, x1.x, x1.y);
                mma_bf16_16816(acc[m][j], wa[m][1].z, wb[m][1].z, wa[m][1].w, wb[m][1].w, x1.z, x1.w);
            }
        }
    }

    // partial sums of the 8 warps, added in warp order
    float4* mine = reinterpret_cast<float4*>(red) + (size_t)warp * (MT * NT * 32);
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < NT; ++j)
            mine[(m * NT + j) * 32 + lane] =
                make_float4(acc[m][j][0], acc[m][j][1], acc[m][j][2], acc[m][j][3]);
    __syncthreads();
    float4* peers = reinterpret_cast<float4*>(red) + (size_t)8 * (MT * NT * 32);
    if (ksplit > 1) {
        asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory");   // (all are running)
        // the blocks of a cluster took alternating runs of k of the same weight rows:
        // each adds its 8 warps and hands the sum to the first block
        if (rank > 0) {
            float4* remote = cluster.map_shared_rank(peers, 0) + (size_t)(rank - 1) * (MT * NT * 32);
            for (int idx = threadIdx.x; idx < MT * NT * 32; idx += blockDim.x) {
                float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int w = 0; w < 8; ++w) {
                    const float4 v =
                        reinterpret_cast<const float4*>(red)[(size_t)w * (MT * NT * 32) + idx];
                    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
                }
                remote[idx] = s;
            }
        }
        cluster.sync();
        if (rank > 0) return;
    }
    for (int idx = threadIdx.x; idx < MT * NT * 32; idx += blockDim.x) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int w = 0; w < 8; ++w) {
            const float4 v = reinterpret_cast<const float4*>(red)[(size_t)w * (MT * NT * 32) + idx];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        for (int b = 1; b < ksplit; ++b) {     // in block order
            const float4 v = peers[(size_t)(b - 1) * (MT * NT * 32) + idx];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        const int l2 = idx & 31, j = (idx >> 5) % NT, m = idx / (32 * NT);
        const int gg = l2 >> 2, tt = l2 & 3;
        const int n_lo = n0 + 16 * m + gg;          // s.x, s.y; n_lo + 8: s.z, s.w
        const int r0 = 8 * j + 2 * tt;              // s.x, s.z; r0 + 1: s.y, s.w
        if (EPI == EPI_ROPE) {
            // s.x, s.y: feature run_a + gg of rows r0, r0 + 1; s.z, s.w: feature run_b + gg
            const int hd = rope.head_dim;
            const int head = run_a / hd, dim = run_a % hd + gg;
            const bool rotates = head < rope.n_heads + rope.n_kv;
            const float in_a[2] = {s.x, s.y}, in_b[2] = {s.z, s.w};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int r = r0 + e;
                if (r >= R) continue;
                const int pos = rope.row_pos[r];
                float oa = in_a[e], ob = in_b[e];
                if (rotates) {
                    const float ang = (float)pos * rope.inv_freq[dim];
                    const float c = cosf(ang), sn = sinf(ang);
                    oa = in_a[e] * c - in_b[e] * sn;
                    ob = in_a[e] * sn + in_b[e] * c;
                }
                y[(size_t)r * y_stride + run_a + gg] = from_f32<OutT>(oa);
                y[(size_t)r * y_stride + run_b + gg] = from_f32<OutT>(ob);
                if (head >= rope.n_heads && rope.k_pool) {
                    const int b = rope.row_seq[r];
                    int cell = pos;
                    bool keep = rope.seq_slot[b] >= 0;     // (a padding row's sequence holds no slot)
                    if (keep && rope.ring_tokens > 0) {
                        keep = pos >= rope.seq_end[b] - rope.ring_tokens;
                        cell = pos % rope.ring_tokens;
                    }
                    if (keep) {
                        const int page = rope.page_table[(size_t)rope.seq_slot[b] * rope.max_pages +
                                                         cell / rope.page_tokens];
                        const bool is_k = head < rope.n_heads + rope.n_kv;
                        const int kvh = head - rope.n_heads - (is_k ? 0 : rope.n_kv);
                        __nv_bfloat16* dst = (is_k ? rope.k_pool : rope.v_pool) +
                            (((size_t)page * rope.n_kv + kvh) * rope.page_tokens + cell % rope.page_tokens) * hd;
                        dst[run_a % hd + gg] = __float2bfloat16(oa);
                        dst[run_b % hd + gg] = __float2bfloat16(ob);
                    }
                }
            }
        } else if (EPI == EPI_GEGLU) {
            // rows gg (gate) and gg + 8 (up) of the 16-row group make column n_out
            const int n_out = (n0 + 16 * m) / 2 + gg;
            if (n_lo + 8 < N) {
                if (r0 < R) y[(size_t)r0 * y_stride + n_out] = from_f32<OutT>(gelu_tanh_f(s.x) * s.z);
                if (r0 + 1 < R)
                    y[(size_t)(r0 + 1) * y_stride + n_out] = from_f32<OutT>(gelu_tanh_f(s.y) * s.w);
            }
        } else {
            float o[4] = {s.x, s.y, s.z, s.w};
            if (EPI == EPI_SOFTCAP) {
#pragma unroll
                for (int c = 0; c < 4; ++c) o[c] = cap * tanhf(o[c] / cap);
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int n = n_lo + (c >= 2 ? 8 : 0), r = r0 + (c & 1);
                if (n < N && r < R) y[(size_t)r * y_stride + n] = from_f32<OutT>(o[c]);
            }
        }
    }
}

template <int NT, int MT, typename OutT, int EPI>
__global__ void __launch_bounds__(256)
skinny_linear_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x,
                     OutT* __restrict__ y, int R, int N, int K, int x_stride, int y_stride,
                     float cap, int ksplit, RopeTail rope) {
    skinny_linear_body<NT, MT, OutT, EPI>(W, x, y, R, N, K, x_stride, y_stride, cap, ksplit, rope);
}

// The same with 48 registers instead of 52 to 56, so that an SM holds five blocks, not four
// (one tile of rows only).
template <typename OutT, int EPI>
__global__ void __launch_bounds__(256, 5)
skinny_linear_dense_kernel(const __nv_bfloat16* __restrict__ W, const __nv_bfloat16* __restrict__ x,
                           OutT* __restrict__ y, int R, int N, int K, int x_stride, int y_stride,
                           float cap, int ksplit, RopeTail rope) {
    skinny_linear_body<1, 1, OutT, EPI>(W, x, y, R, N, K, x_stride, y_stride, cap, ksplit, rope);
}

template <int NT, int MT, typename OutT, int EPI>
static int launch_skinny(const void* W, const void* x, void* y, int R, int N, int K, int x_stride,
                         int y_stride, float cap, const RopeTail& rope, cudaStream_t s) {
    const int blocks = (N + 16 * MT - 1) / (16 * MT);
    // few weight rows: several blocks (a cluster) share a tile of rows and split k, so
    // that enough loads are in flight to fill the memory system
    static int sms = 0;          // (of the first device asked: the split is a matter of speed only)
    if (!sms) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
            sms = 148;
    }
    static const int fill = getenv("SIB_SKINNY_FILL") ? atoi(getenv("SIB_SKINNY_FILL")) : 3;
    int ksplit = 1;
    while (ksplit < 8 && blocks * ksplit < fill * sms && K >= 2 * ksplit * 8 * 64) ksplit *= 2;
    const size_t smem = (size_t)(8 + ksplit - 1) * MT * NT * 32 * 4 * sizeof(float);
    // Five blocks an SM instead of four (48 registers, which costs a warp some of the loads
    // it keeps in flight) where that is what lets every block be resident at once: a grid
    // that nearly fills or overflows four blocks an SM and fits five.  Clusters need their
    // blocks' places free at the same time, so a nearly full device places the last ones late.
    // (Measured on single-token steps at context 8 192, batch 8 / batch 1: the Gemma2-2B shape's
    // output and down products, 576 blocks each, -2.8 % / -5.7 % of the step's time, with q|k|v's
    // 512 blocks -2.8 % / -6.3 %; its gate/up product, 1 152 blocks, +0.4 % / +1.1 %; the 9B shape's
    // output product, 448 blocks, +0.9 % / +1.8 %; every product of the 27B shape +3.2 % / +5.6 %,
    // its down product with 18 432 of k a block most of it: so only blocks with a short run of k.)
    static const int dense_k = getenv("SIB_SKINNY_DENSE_K") ? atoi(getenv("SIB_SKINNY_DENSE_K")) : 2560;
    const long long grid_blocks = (long long)blocks * ksplit;
    bool dense = NT == 1 && MT == 1 && 20 * grid_blocks > 17 * 4 * sms && grid_blocks <= 5 * sms &&
                 K / ksplit <= dense_k;
    if (const char* only = getenv("SIB_SKINNY_DENSE_SHAPES")) {      // (for measurements)
        char want[64];
        snprintf(want, sizeof want, "%dx%d", N, K);
        dense = NT == 1 && MT == 1 && (strstr(only, want) != nullptr || strstr(only, "all") != nullptr);
    }
    auto kernel = dense ? skinny_linear_dense_kernel<OutT, EPI> : skinny_linear_kernel<NT, MT, OutT, EPI>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) {
            sib_set_error("skinny_linear: shared memory: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(blocks, ksplit, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = ksplit;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sib_chained_launches() ? 2 : 1;
    sib_same_carveout(kernel);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, (const __nv_bfloat16*)W,
                                       (const __nv_bfloat16*)x, (OutT*)y, R, N, K, x_stride,
                                       y_stride, cap, ksplit, rope);
    if (e != cudaSuccess) {
        sib_set_error("skinny_linear: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return sib_check_launch("skinny_linear");
}

template <typename OutT, int EPI>
static int dispatch_skinny(const void* W, const void* x, void* y, int R, int N, int K,
                           int x_stride, int y_stride, float cap, const RopeTail& rope,
                           cudaStream_t s) {
#define GO(NT, MT) \
    return launch_skinny<NT, MT, OutT, EPI>(W, x, y, R, N, K, x_stride, y_stride, cap, rope, s)
    if (R <= 8) GO(1, 1);
    if (R <= 16) GO(2, 1);
    if constexpr (EPI == EPI_ROPE) {
        sib_set_error("skinny_linear: the rotating product takes at most 16 rows, not %d", R);
        return -1;
    } else {
        if (R <= 32) GO(4, 2);
        GO(8, 2);
    }
#undef GO
}

// The largest R this kernel takes.
SIB_EXPORT int sib_skinny_linear_max_rows() { return 64; }

SIB_EXPORT int sib_skinny_linear(const void* W, const void* x, void* y, int out_dtype, int R, int N,
                                 int K, int x_stride, int y_stride, int epilogue, float cap,
                                 void* stream) {
    if (R == 0) return 0;
    SIB_REQUIRE(R > 0 && R <= 64, "skinny_linear: %d rows; this kernel takes 1 to 64", R);
    SIB_REQUIRE(N > 0 && K > 0 && K % 8 == 0,
                "skinny_linear: N=%d K=%d; K must be a multiple of 8", N, K);
    SIB_REQUIRE(x_stride % 8 == 0 && ((uintptr_t)W % 16) == 0 && ((uintptr_t)x % 16) == 0,
                "skinny_linear: operands must be 16-byte aligned (x_stride=%d)", x_stride);
    SIB_REQUIRE(epilogue != EPI_GEGLU || N % 16 == 0,
                "skinny_linear: the gated epilogue needs N (%d) in whole groups of 16", N);
    SIB_REQUIRE(epilogue != EPI_SOFTCAP || cap > 0.f, "skinny_linear: soft cap must be positive");
    cudaStream_t s = (cudaStream_t)stream;
#define GO(OUT, EPI) \
    return dispatch_skinny<OUT, EPI>(W, x, y, R, N, K, x_stride, y_stride, cap, RopeTail{}, s)
    if (out_dtype == SIB_BF16) {
        if (epilogue == EPI_NONE) GO(__nv_bfloat16, EPI_NONE);
        if (epilogue == EPI_GEGLU) GO(__nv_bfloat16, EPI_GEGLU);
        if (epilogue == EPI_SOFTCAP) GO(__nv_bfloat16, EPI_SOFTCAP);
    } else if (out_dtype == SIB_F32) {
        if (epilogue == EPI_NONE) GO(float, EPI_NONE);
        if (epilogue == EPI_SOFTCAP) GO(float, EPI_SOFTCAP);
        if (epilogue == EPI_GEGLU) GO(float, EPI_GEGLU);
    }
#undef GO
    SIB_REQUIRE(false, "skinny_linear: unknown output type %d or epilogue %d", out_dtype, epilogue);
}


// The q|k|v product of attention for at most 16 rows, followed in the same kernel by what
// sib_rope_store does (half-split pairing over the whole head): y[R, (n_heads + 2 n_kv) *
// head_dim] gets q and k rotated and v, and k and v also go into the paged cache.
// n_kv == 0: W holds the q rows only and nothing is stored.
SIB_EXPORT int sib_skinny_linear_rope(const void* W, const void* x, void* y, int R, int K,
                                      int x_stride, int y_stride, const int* row_pos,
                                      const int* row_seq, const int* seq_slot, const int* seq_end,
                                      const float* inv_freq, void* k_pool, void* v_pool,
                                      const int* page_table, int max_pages, int page_tokens,
                                      int ring_tokens, int n_heads, int n_kv, int head_dim,
                                      void* stream) {
    if (R == 0) return 0;
    SIB_REQUIRE(R > 0 && R <= 16, "skinny_linear_rope: %d rows; this product takes 1 to 16", R);
    SIB_REQUIRE(n_heads > 0 && n_kv >= 0 && head_dim > 0 && head_dim % 16 == 0,
                "skinny_linear_rope: heads=%d kv=%d head_dim=%d (a multiple of 16)", n_heads, n_kv,
                head_dim);
    SIB_REQUIRE(K > 0 && K % 8 == 0 && x_stride % 8 == 0 && ((uintptr_t)W % 16) == 0 &&
                    ((uintptr_t)x % 16) == 0,
                "skinny_linear_rope: K=%d and the operands must be aligned to 8 elements", K);
    SIB_REQUIRE(row_pos && inv_freq, "skinny_linear_rope: positions and frequencies are needed");
    SIB_REQUIRE(n_kv == 0 || (k_pool && v_pool && page_table && row_seq && seq_slot && seq_end &&
                              page_tokens > 0 && max_pages > 0),
                "skinny_linear_rope: incomplete cache description");
    SIB_REQUIRE(ring_tokens >= 0 && (ring_tokens == 0 || ring_tokens % page_tokens == 0),
                "skinny_linear_rope: ring of %d tokens is not whole pages of %d", ring_tokens,
                page_tokens);
    const int N = (n_heads + 2 * n_kv) * head_dim;
    RopeTail rope{row_pos, row_seq, seq_slot, seq_end, inv_freq,
                  n_kv ? (__nv_bfloat16*)k_pool : nullptr, (__nv_bfloat16*)v_pool, page_table,
                  n_heads, n_kv, head_dim, max_pages, page_tokens, ring_tokens};
    return dispatch_skinny<__nv_bfloat16, EPI_ROPE>(W, x, y, R, N, K, x_stride, y_stride, 0.f, rope,
                                                    (cudaStream_t)stream);
}
