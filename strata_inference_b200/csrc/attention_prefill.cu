// Attention of whole prompts over the step's own keys and values (bfloat16):
// the compute-bound kernel of prefill, in the manner of flash attention.
// Same mathematics as attention_rows.cu (scale, soft cap, causal and window
// mask, softmax in 32-bit, weighted sum of v).
//
// A block of 4 warps takes 64 query rows of one (sequence, kv head): the G
// query heads that share the kv head times 64 / G consecutive positions, so a
// key/value tile is loaded once for all of them.  Keys are walked in tiles of
// 64, from the first tile any of its rows can see (window) to the diagonal
// (causal); tiles are copied into shared memory with cp.async, two tiles in
// flight, 16-byte chunks XOR-swizzled by row so that ldmatrix reads are free
// of bank conflicts.  Scores and the weighted sum run on mma.m16n8k16 with the
// output accumulator in registers; probabilities never leave registers.
//
// Plain counterpart: tests/plain_gemma2.py attention().
// Reference: src/backend/cuda/kernels.rs:3183-3430 (batched_causal_attention:
// one block per (head, query), online softmax over key tiles of 256).
#include "common.cuh"

struct AttnPrefillArgs {
    const __nv_bfloat16* qkv;   // packed rows [q heads | k heads | v heads], rotated
    __nv_bfloat16* out;         // [rows, n_heads * head_dim]
    const int* seq_row0;        // [seqs] first packed row of the sequence
    const int* seq_len;         // [seqs] rows (= positions, the step starts at position 0)
    int width;                  // elements per packed row
    int n_heads, n_kv;
    int window;
    float scale, softcap;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;   // 0: the chunk is filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* smem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// tanh on the special-function unit (relative error about 2^-11: below the 2^-9 of the
// bfloat16 operands the scores were computed from).
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Element (row, col) of a tile whose rows hold HD bfloat16 in swizzled 16-byte chunks.
template <int HD>
__device__ __forceinline__ __nv_bfloat16* tile_at(__nv_bfloat16* tile, int row, int chunk) {
    return tile + row * HD + ((chunk ^ (row & 7)) << 3);
}

template <int HD>
__device__ __forceinline__ void load_rows(__nv_bfloat16* tile, const __nv_bfloat16* src, int width,
                                          int first_row, int n_rows_valid) {
    // 64 rows x HD/8 chunks, spread over 128 threads
    constexpr int CH = HD / 8;
    for (int i = threadIdx.x; i < 64 * CH; i += 128) {
        const int row = i / CH, chunk = i % CH;
        const bool ok = row < n_rows_valid;
        const __nv_bfloat16* g = src + (size_t)(first_row + (ok ? row : 0)) * width + chunk * 8;
        cp_async16(tile_at<HD>(tile, row, chunk), g, ok);
    }
}

// HD: head size (64, 128, 256).  G: query heads per kv head (1, 2, 4).
template <int HD, int G>
__global__ void __launch_bounds__(128) attention_prefill_kernel(AttnPrefillArgs p) {
    constexpr int MP = 64 / G;           // positions per block
    constexpr int KS = HD / 16;          // k-steps of the score product
    constexpr int DN = HD / 8;           // n-tiles of the output
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    // Two key/value tiles in flight where two blocks per SM still fit (heads up to 128);
    // one tile for wider heads, where the second block of the SM hides the loads instead.
    constexpr bool DOUBLE = HD <= 128;
    constexpr int NBUF = DOUBLE ? 2 : 1;
    __nv_bfloat16* Ks = Qs + 64 * HD;
    __nv_bfloat16* Vs = Ks + NBUF * 64 * HD;

    const int b = blockIdx.y, kvh = blockIdx.z;
    const int n = p.seq_len[b];
    // late tiles see the most keys: they go first, so that the short ones fill the tail
    const int p0 = (int)(gridDim.x - 1 - blockIdx.x) * MP;
    if (p0 >= n) return;
    const int row0 = p.seq_row0[b];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;

    // ---- the query tile: row i = head (i / MP) of the group, position p0 + i % MP ----
    {
        constexpr int CH = HD / 8;
        for (int i = threadIdx.x; i < 64 * CH; i += 128) {
            const int row = i / CH, chunk = i % CH;
            const int pos = p0 + row % MP;
            const bool ok = pos < n;
            const int head = kvh * G + row / MP;
            const __nv_bfloat16* src =
                p.qkv + (size_t)(row0 + (ok ? pos : 0)) * p.width + (size_t)head * HD + chunk * 8;
            cp_async16(tile_at<HD>(Qs, row, chunk), src, ok);
        }
    }
    const int k_hi = min(n, p0 + MP);                                    // keys < k_hi
    const int k_lo = p.window > 0 ? max(0, p0 - p.window + 1) : 0;
    const int kt0 = k_lo >> 6, kt1 = (k_hi + 63) >> 6;
    const __nv_bfloat16* kbase = p.qkv + (size_t)row0 * p.width + (size_t)(p.n_heads + kvh) * HD;
    const __nv_bfloat16* vbase = kbase + (size_t)p.n_kv * HD;
    load_rows<HD>(Ks, kbase, p.width, kt0 * 64, n - kt0 * 64);
    if (!DOUBLE) cp_async_commit();              // queries and keys first, values as a second group
    load_rows<HD>(Vs, vbase, p.width, kt0 * 64, n - kt0 * 64);
    cp_async_commit();

    float o[DN][4];
#pragma unroll
    for (int d = 0; d < DN; ++d) o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // positions of this lane's two rows (g and g + 8 of the warp's 16)
    const int qpos0 = p0 + (16 * warp + g) % MP, qpos1 = p0 + (16 * warp + g + 8) % MP;

    for (int kt = kt0; kt < kt1; ++kt) {
        const int buf = DOUBLE ? (kt - kt0) & 1 : 0;
        if (DOUBLE) {
            if (kt + 1 < kt1) {
                load_rows<HD>(Ks + (buf ^ 1) * 64 * HD, kbase, p.width, (kt + 1) * 64, n - (kt + 1) * 64);
                load_rows<HD>(Vs + (buf ^ 1) * 64 * HD, vbase, p.width, (kt + 1) * 64, n - (kt + 1) * 64);
                cp_async_commit();
                cp_async_wait<1>();
            } else {
                cp_async_wait<0>();
            }
        } else {
            if (kt > kt0) {
                load_rows<HD>(Ks, kbase, p.width, kt * 64, n - kt * 64);
                cp_async_commit();
                load_rows<HD>(Vs, vbase, p.width, kt * 64, n - kt * 64);
                cp_async_commit();
            }
            cp_async_wait<1>();                  // the keys (and the queries) are here
        }
        __syncthreads();
        __nv_bfloat16* Kt = Ks + buf * 64 * HD;
        __nv_bfloat16* Vt = Vs + buf * 64 * HD;

        // ---- scores of 16 rows x 64 keys ----
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            uint32_t a[4];
            ldsm_x4(a, tile_at<HD>(Qs, 16 * warp + (lane & 15), 2 * ks + (lane >> 4)));
#pragma unroll
            for (int jp = 0; jp < 4; ++jp) {       // pairs of 8-key tiles
                uint32_t kb[4];
                const int mi = lane >> 3;
                ldsm_x4(kb, tile_at<HD>(Kt, 16 * jp + (mi >> 1) * 8 + (lane & 7), 2 * ks + (mi & 1)));
                mma_16816(s[2 * jp], a, kb[0], kb[1]);
                mma_16816(s[2 * jp + 1], a, kb[2], kb[3]);
            }
        }
        // ---- scale, cap, mask, online softmax ----
        // Most tiles lie wholly below the diagonal and inside the window of all 16 rows
        // of the warp (consecutive positions of one head): no per-element mask there.
        const int wq_lo = p0 + (16 * warp) % MP;
        const bool inside = kt * 64 + 63 <= wq_lo && kt * 64 + 63 < n &&
                            (p.window <= 0 || wq_lo + 15 - kt * 64 < p.window);
        const float inv_cap = p.softcap > 0.f ? 1.0f / p.softcap : 0.f;
        float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v = s[j][i] * p.scale;
                if (p.softcap > 0.f) v = p.softcap * tanh_fast(v * inv_cap);
                if (!inside) {
                    const int key = kt * 64 + 8 * j + 2 * t + (i & 1);
                    const int qp = (i < 2) ? qpos0 : qpos1;
                    const bool seen = key <= qp && key < n && (p.window <= 0 || qp - key < p.window);
                    v = seen ? v : -INFINITY;
                }
                s[j][i] = v;
                mx[i >> 1] = fmaxf(mx[i >> 1], v);
            }
        }
        float corr[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            m_use[r] = mx[r] == -INFINITY ? 0.f : mx[r];     // a row that has seen no key yet
            corr[r] = __expf(m_run[r] - m_use[r]);
            m_run[r] = mx[r];
            l_run[r] *= corr[r];
        }
#pragma unroll
        for (int d = 0; d < DN; ++d) {
            o[d][0] *= corr[0]; o[d][1] *= corr[0];
            o[d][2] *= corr[1]; o[d][3] *= corr[1];
        }
        float lsum[2] = {0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float e = __expf(s[j][i] - m_use[i >> 1]);
                s[j][i] = e;
                lsum[i >> 1] += e;
            }
        }
        l_run[0] += lsum[0];
        l_run[1] += lsum[1];
        if (!DOUBLE) {
            cp_async_wait<0>();                  // the values are here
            __syncthreads();
        }
        // ---- weighted sum: 16 keys per k-step, probabilities as the A operand ----
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
            uint32_t a[4];
            a[0] = pack_bf16(s[2 * jj][0], s[2 * jj][1]);
            a[1] = pack_bf16(s[2 * jj][2], s[2 * jj][3]);
            a[2] = pack_bf16(s[2 * jj + 1][0], s[2 * jj + 1][1]);
            a[3] = pack_bf16(s[2 * jj + 1][2], s[2 * jj + 1][3]);
#pragma unroll
            for (int dn = 0; dn < HD / 16; ++dn) {
                uint32_t vb[4];
                const int mi = lane >> 3;
                ldsm_x4_trans(vb, tile_at<HD>(Vt, 16 * jj + (mi & 1) * 8 + (lane & 7),
                                              2 * dn + (mi >> 1)));
                mma_16816(o[2 * dn], a, vb[0], vb[1]);
                mma_16816(o[2 * dn + 1], a, vb[2], vb[3]);
            }
        }
        __syncthreads();   // the other buffer is overwritten by the next iteration's loads
    }

    // ---- normalise and store ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = 16 * warp + g + 8 * r;
        const int pos = p0 + row % MP;
        if (pos >= n) continue;
        const int head = kvh * G + row / MP;
        const float inv = 1.0f / l_run[r];
        __nv_bfloat16* dst = p.out + (size_t)(row0 + pos) * p.n_heads * HD + (size_t)head * HD;
#pragma unroll
        for (int d = 0; d < DN; ++d) {
            *reinterpret_cast<uint32_t*>(dst + 8 * d + 2 * t) =
                pack_bf16(o[d][2 * r] * inv, o[d][2 * r + 1] * inv);
        }
    }
}

SIB_EXPORT int sib_attention_prefill_supports(int n_heads, int n_kv, int head_dim) {
    if (n_kv <= 0 || n_heads % n_kv) return 0;
    const int G = n_heads / n_kv;
    return (G == 1 || G == 2 || G == 4) && (head_dim == 64 || head_dim == 128 || head_dim == 256);
}

template <int HD, int G>
static int launch_prefill(const AttnPrefillArgs& p, int n_seqs, int max_len, cudaStream_t s) {
    const size_t smem = (size_t)(HD <= 128 ? 5 : 3) * 64 * HD * sizeof(__nv_bfloat16);
    auto kernel = attention_prefill_kernel<HD, G>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) {
            sib_set_error("attention_prefill: shared memory: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    constexpr int MP = 64 / G;
    dim3 grid((max_len + MP - 1) / MP, n_seqs, p.n_kv);
    kernel<<<grid, 128, smem, s>>>(p);
    return sib_check_launch("attention_prefill");
}

// Attention of `n_seqs` packed prompts that all start at position 0.
SIB_EXPORT int sib_attention_prefill(const void* qkv, int width, void* out, const int* seq_row0,
                                     const int* seq_len, int n_seqs, int max_len, int n_heads,
                                     int n_kv, int head_dim, float scale, float softcap,
                                     int window, void* stream) {
    if (n_seqs == 0 || max_len == 0) return 0;
    SIB_REQUIRE(sib_attention_prefill_supports(n_heads, n_kv, head_dim),
                "attention_prefill: heads=%d kv_heads=%d head_dim=%d is not a shape this kernel "
                "takes (groups of 1, 2 or 4 heads; head_dim 64, 128 or 256)",
                n_heads, n_kv, head_dim);
    SIB_REQUIRE(width == (n_heads + 2 * n_kv) * head_dim && ((uintptr_t)qkv % 16) == 0 &&
                    ((uintptr_t)out % 16) == 0,
                "attention_prefill: packed rows of %d elements do not fit the head counts", width);
    SIB_REQUIRE(n_seqs > 0 && n_seqs < 65536 && n_kv < 65536 && max_len > 0 && window >= 0,
                "attention_prefill: seqs=%d max_len=%d", n_seqs, max_len);
    AttnPrefillArgs p{(const __nv_bfloat16*)qkv, (__nv_bfloat16*)out, seq_row0, seq_len, width,
                      n_heads, n_kv, window, scale, softcap};
    cudaStream_t s = (cudaStream_t)stream;
    const int G = n_heads / n_kv;
#define BY_G(HD)                                                              \
    do {                                                                      \
        if (G == 1) return launch_prefill<HD, 1>(p, n_seqs, max_len, s);      \
        if (G == 2) return launch_prefill<HD, 2>(p, n_seqs, max_len, s);      \
        return launch_prefill<HD, 4>(p, n_seqs, max_len, s);                  \
    } while (0)
    if (head_dim == 64) BY_G(64);
    if (head_dim == 128) BY_G(128);
    BY_G(256);
#undef BY_G
}
