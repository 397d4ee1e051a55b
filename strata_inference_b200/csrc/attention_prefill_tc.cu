// Attention of whole prompts on the fifth-generation tensor cores (bfloat16):
// both products of flash attention as tcgen05.mma with the score tile, the
// probabilities and the output accumulator in tensor memory.  Same mathematics as
// attention_rows.cu (scale, soft cap, causal and window mask, softmax in 32-bit,
// weighted sum of v); attention_prefill.cu is the mma.sync kernel this one
// supersedes where its shapes fit (1 or 2 query heads per kv head, head size 64,
// 128 or 256).
//
// A block takes 128 query rows of one (sequence, kv head): G heads x 128/G
// consecutive positions.  Keys and values are walked in tiles of 128 positions.
// Tensor memory (512 columns): two score tiles S0, S1 of 128 columns, then O.
//
//   warp 0      TMA: the query tile once, then key and value tiles (one of each in
//               flight for head size 256, two for smaller heads), straight from the
//               step's packed q|k|v rows (boxes of 64 rows x 64 columns, 128-byte swizzle)
//   warp 1      one lane issues S(t+1) = Q K^T (128 x 128, operands K-major in shared
//               memory) while the softmax warps work on S(t), and O += P(t) V (128 x
//               head_dim; P read from tensor memory, V the MN-major operand: its rows
//               are keys, as they lie in memory) once P(t) is there
//   warps 2-9   two threads per query row, 64 of the tile's keys each: read S from
//               tensor memory, scale, cap, mask, exponentiate against a running
//               maximum the two agree on, and write P (bfloat16) over the first columns
//               of the same score tile; at the end read O, divide by the row sum, store
//
// The tensor pipe runs what one thread issues in order, so S(t+2) is not written
// before P(t) V has read P(t) from the same columns.
// The running maximum is only raised (and O rescaled in tensor memory) when a
// row's maximum has grown by more than 8 in units of log 2: until then probabilities
// may exceed 1 by at most 2^8, which bfloat16 and the 32-bit sums hold easily, and the
// division by the row sum at the end makes the result the same.
// Every mbarrier wait is bounded; a wait that runs out sets an error flag.
//
// Plain counterpart: tests/plain_gemma2.py attention().
// Reference: src/backend/cuda/kernels.rs:3183-3430 (batched_causal_attention).
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <queue>
#include <vector>

#include "common.cuh"

namespace {

constexpr int BM = 128;   // query rows per block
constexpr int BN = 128;   // keys per tile
constexpr uint32_t WAIT_LIMIT = 1u << 22;

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
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(bar)) : "memory");
}
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
// K-major operand: rows of 128 bytes (64 elements of k), 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_k_major(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) >> 4) & 0x3FFF);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// MN-major operand: rows are k (keys), 64 elements of n (128 bytes) per row; 8-row groups
// 1024 bytes apart along k, blocks of 64 n `n_block_bytes` apart.
__device__ __forceinline__ uint64_t desc_mn_major(const void* tile, uint32_t n_block_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) >> 4) & 0x3FFF);
    d |= (uint64_t)((n_block_bytes >> 4) & 0x3FFF) << 16;
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
// the A operand from tensor memory (128 lanes x 8 columns: 16 bfloat16 of k per lane)
__device__ __forceinline__ void umma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b,
                                             uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate)
        : "memory");
}
// ---- the same on a pair of blocks (a cluster of two, tcgen05 cta_group::2) ----
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
__device__ __forceinline__ void umma_bf16_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b,
                                                  uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate)
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
__device__ __forceinline__ void mbar_arrive_first_block(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];\n" ::"r"(in_first_block(bar))
                 : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                     smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t* r) {
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
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    tmem_ld32_issue(taddr, r);
    tmem_ld_wait();
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
        "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
        "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ float tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Whether key j of the thread's 64 keys is one the row sees.
__device__ __forceinline__ bool sees(int j, int j_lo, int j_hi) { return j >= j_lo && j <= j_hi; }

// The largest of 64 raw products (of those the row sees, with MASK).
template <bool MASK>
__device__ __forceinline__ float row_max(const uint32_t (&raw)[64], int j_lo, int j_hi) {
    float m[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 64; ++j) {
        float v = __uint_as_float(raw[j]);
        if (MASK) v = sees(j, j_lo, j_hi) ? v : -INFINITY;
        m[j & 3] = fmaxf(m[j & 3], v);
    }
    return fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3]));
}

// 64 probabilities 2^(score - ref) as 32 packed bfloat16 pairs (in place of the raw
// products); returns their sum.  CAP: score = c2 * tanh(product * c1), else product * c1.
template <bool CAP, bool MASK>
__device__ __forceinline__ float probabilities(uint32_t (&raw)[64], float c1, float c2, float ref,
                                               int j_lo, int j_hi) {
    float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        float e[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int j = 2 * k + h;
            float x = __uint_as_float(raw[j]);
            if (CAP) x = fmaf(c2, tanh_fast(x * c1), -ref);
            else x = fmaf(x, c1, -ref);
            if (MASK) x = sees(j, j_lo, j_hi) ? x : -INFINITY;
            e[h] = exp2_fast(x);
        }
        sum[k & 3] += e[0] + e[1];
        raw[k] = pack_bf16(e[0], e[1]);       // slot k <= 2k: not read again
    }
    return (sum[0] + sum[1]) + (sum[2] + sum[3]);
}

struct TcArgs {
    __nv_bfloat16* out;      // [rows, n_heads * head_dim]
    const int* seq_row0;
    const int* seq_len;
    const int* seq_q0;       // per sequence: rows before this position are keys only (null: none)
    int* error_flag;
    float* part;             // partial results of split blocks (see SPLIT below), or null
    int* tickets;            // 8 per block of query rows, zero between launches
    int split_tiles;         // blocks with at least this many key tiles are split (0: none)
    int n_heads, n_kv;
    int window;
    float scale, softcap;
};

// SPLIT.  When the grid is small against the device, a block (or pair) of query rows with
// many key tiles is run twice, by blockIdx.z / n_kv = 0 and 1, each over half of the
// tiles.  Both write max, sum and accumulator of their rows to `part`, warp by warp,
// then draw a ticket of that warp's rows; the warp that draws the second ticket adds the
// other's partial result to its own and stores the output.
// Floats of `part` for one block of 128 query rows and one half:
template <int HD>
__host__ __device__ constexpr size_t part_floats() { return (size_t)BM * (HD + 2); }

// BALANCE.  When the host knows the prompts' lengths, a launch is a list of work items
// instead of a grid over (block of query rows, sequence, kv head): one item per block (or
// pair) of query rows, or two for a block whose run of key tiles is split, ordered by the
// work in them, longest first, so that blocks are handed to the SMs in that order.  Which
// blocks are split is what makes the longest SM's share smallest (plan_items below).
constexpr int MAX_ITEMS = 384;
struct TcItems {
    int n;                       // 0: the launch is a grid (see the kernel)
    uint32_t where[MAX_ITEMS];   // sequence << 20 | kv head << 12 | block of query rows (of NB * MP positions)
    uint32_t what[MAX_ITEMS];    // split unit (0xFFFFFF: not split) | part << 24
};

// Barriers of one block.
struct Bars {
    uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], p_full[2], pair[4],
        pv_done, o_done;
};

}  // namespace

// PAIR: two blocks (a cluster) take 256 query rows, two neighbouring runs of positions,
// and share every key and value tile: each loads 64 of the tile's 128 keys and half of
// the value columns, and one thread of the first block issues the MMAs for both
// (cta_group::2, M = 256), so a tile crosses from L2 once per pair and the halved tiles
// leave room for two of each in flight at head size 256.
template <int HD, int G, bool PAIR>
__global__ void __launch_bounds__(320)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map, TcArgs p,
                            const __grid_constant__ TcItems items) {
    static_assert(!PAIR || HD >= 128, "half of the value columns must fill a 128-byte row");
    constexpr int MP = BM / G;                 // positions per block
    constexpr int CH = HD / 64;                // 64-wide column chunks of a head
    constexpr int ST = (HD == 256 && !PAIR) ? 1 : 2;   // key tiles (and value tiles) in flight
    constexpr int NB = PAIR ? 2 : 1;           // blocks that share the tiles
    constexpr int K_ROWS = BN / NB;            // keys of a tile in this block's shared memory
    constexpr int V_CH = CH / NB;              // 64-column chunks of the values here
    constexpr uint32_t Q_BYTES = BM * HD * 2, KV_BYTES = BN * HD * 2 / NB;
    constexpr uint32_t K_CHUNK = K_ROWS * 128; // one 64-column chunk of this block's keys
    constexpr uint32_t V_CHUNK = BN * 128;     // one 64-column chunk of a value tile
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t O_COL = 256;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* Qs = base;                              // CH chunks of [128 rows x 128 B]
    unsigned char* Ks = Qs + Q_BYTES;                      // ST stages of CH chunks of [128 x 128 B]
    unsigned char* Vs = Ks + ST * KV_BYTES;                // the same
    Bars* bars = reinterpret_cast<Bars*>(Vs + ST * KV_BYTES);
    float* xch = reinterpret_cast<float*>(bars + 1);       // [2 tiles][2 halves][128 rows]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xch + 2 * 2 * BM);
    int* failed = reinterpret_cast<int*>(tmem_slot + 1);

    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = PAIR ? (int)cluster_ctarank() : 0;
    int b, kvh, part, first0;           // first0: the first position of the block or of the pair
    size_t unit = 0;                    // which pair of partial results a split block uses
    bool listed_split = false;
    if (items.n > 0) {
        const uint32_t where = items.where[blockIdx.x / NB], what = items.what[blockIdx.x / NB];
        b = (int)(where >> 20);
        kvh = (int)((where >> 12) & 0xFFu);
        first0 = (int)(where & 0xFFFu) * (NB * MP);
        part = (int)((what >> 24) & 1u);
        listed_split = (what & 0xFFFFFFu) != 0xFFFFFFu;
        unit = (size_t)(what & 0xFFFFFFu) * NB + rank;
    } else {
        b = blockIdx.y;
        kvh = blockIdx.z % p.n_kv;
        part = blockIdx.z / p.n_kv;
        // the longest tiles first
        first0 = (int)(gridDim.x / NB - 1 - blockIdx.x / NB) * (NB * MP);
        unit = ((size_t)b * p.n_kv + kvh) * gridDim.x + blockIdx.x;
    }
    const int n = p.seq_len[b];
    const int q0 = p.seq_q0 ? p.seq_q0[b] : 0;
    const int p0 = first0 + rank * MP;
    if (first0 >= n || first0 + NB * MP <= q0) return;     // (both blocks of a pair)
    const int row0 = p.seq_row0[b];
    const int k_hi = min(n, first0 + NB * MP);
    const int k_lo = p.window > 0 ? max(0, first0 - p.window + 1) : 0;
    int kt0 = k_lo / BN, nt = (k_hi + BN - 1) / BN - kt0;
    // a long run of key tiles is shared with the block that has the other part
    // (the other blockIdx.z / n_kv of a grid, the other item of a list)
    const bool is_split = items.n > 0 ? listed_split : (p.split_tiles > 0 && nt >= p.split_tiles);
    if (part == 1 && !is_split) return;                    // (both blocks of a pair)
    if (is_split) {
        const int first_half = (nt + 1) / 2;
        if (part == 1) kt0 += first_half;
        nt = part == 0 ? first_half : nt - first_half;
    }
    const int q_col = kvh * G * HD;                        // first column of the group's heads
    const int k_col = (p.n_heads + kvh) * HD;
    const int v_col = (p.n_heads + p.n_kv + kvh) * HD;

    if (threadIdx.x == 0) {
        mbar_init(&bars->q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&bars->k_full[s], 1);
            mbar_init(&bars->k_empty[s], 1);
            mbar_init(&bars->v_full[s], 1);
            mbar_init(&bars->v_empty[s], 1);
            mbar_init(&bars->s_full[s], 1);
            mbar_init(&bars->p_full[s], 8 * NB);       // the softmax warps of every block
        }
        for (int q = 0; q < 4; ++q) mbar_init(&bars->pair[q], 2);
        mbar_init(&bars->pv_done, 1);
        mbar_init(&bars->o_done, 1);
        *failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                             smem_u32(tmem_slot)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(
                             smem_u32(tmem_slot)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync_all();     // both blocks' barriers exist before anything arrives on them
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    // a load whose bytes are counted on the (first block's) barrier; an arrival that
    // announces the bytes of all blocks, by the first block only
    auto load = [&](void* dst, uint64_t* bar, int c0, int c1) {
        if (PAIR) tma_load_2d_pair(dst, &map, bar, c0, c1);
        else tma_load_2d(dst, &map, bar, c0, c1);
    };
    auto expect = [&](uint64_t* bar, uint32_t bytes) {
        if (rank == 0) mbar_arrive_expect_tx(bar, NB * bytes);
    };

    if (warp == 0) {
        if (lane == 0) {
            // Barriers, tensor memory and the roles above needed nothing from the kernel that
            // wrote q, k and v; the loads do.  (Every other thread of the block only ever
            // acts on what these loads bring.)
            pdl_wait();
            // the query tile: per 64-column chunk two boxes of 64 rows
            expect(&bars->q_full, Q_BYTES);
            for (int c = 0; c < CH; ++c)
                for (int half = 0; half < 2; ++half) {
                    const int head = (half * 64) / MP, off = (half * 64) % MP;
                    load(Qs + c * (BM * 128) + half * (64 * 128), &bars->q_full,
                         q_col + head * HD + 64 * c, row0 + p0 + off);
                }
            // A key tile is free again once its scores have been formed, a value tile
            // only after the product that follows them: keys run ahead of values.
            // (of a pair, this block brings keys [64 rank, 64 rank + 64) of a tile, all columns,
            // and all 128 keys' value columns [HD / 2 * rank, HD / 2 * rank + HD / 2))
            auto load_k = [&](int t) -> bool {
                const int s = t % ST;
                if (t >= ST && !mbar_wait(&bars->k_empty[s], ((t / ST) - 1) & 1)) return false;
                expect(&bars->k_full[s], KV_BYTES);
                for (int c = 0; c < CH; ++c)
                    for (int r64 = 0; r64 < K_ROWS / 64; ++r64)
                        load(Ks + s * KV_BYTES + c * K_CHUNK + r64 * (64 * 128), &bars->k_full[s],
                             k_col + 64 * c, row0 + (kt0 + t) * BN + K_ROWS * rank + 64 * r64);
                return true;
            };
            auto load_v = [&](int t) -> bool {
                const int s = t % ST;
                if (t >= ST && !mbar_wait(&bars->v_empty[s], ((t / ST) - 1) & 1)) return false;
                expect(&bars->v_full[s], KV_BYTES);
                for (int c = 0; c < V_CH; ++c)
                    for (int r64 = 0; r64 < BN / 64; ++r64)
                        load(Vs + s * KV_BYTES + c * V_CHUNK + r64 * (64 * 128), &bars->v_full[s],
                             v_col + (HD / NB) * rank + 64 * c, row0 + (kt0 + t) * BN + 64 * r64);
                return true;
            };
            bool fed = nt == 0 || load_k(0);
            for (int t = 0; t < nt && fed; ++t) {
                if (t + 1 < nt) fed = load_k(t + 1);
                fed = fed && load_v(t);
            }
            if (!fed) *failed = 1;
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            // M is 128 rows of one block or 256 rows over the pair
            constexpr uint32_t IDESC_QK = (1u << 4) | (1u << 7) | (1u << 10) |
                                          ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(NB * BM >> 4) << 24);
            constexpr uint32_t IDESC_PV = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                          ((uint32_t)(HD >> 3) << 17) | ((uint32_t)(NB * BM >> 4) << 24);
            auto commit = [&](uint64_t* bar) {
                if (PAIR) umma_commit_pair(bar);
                else umma_commit(bar);
            };
            bool ok = mbar_wait(&bars->q_full, 0);
            if (!ok) *failed = 2;
            // S(t) = Q K(t)^T into score tile t & 1: HD / 16 steps of k
            auto issue_qk = [&](int t) {
                const unsigned char* kt = Ks + (t % ST) * KV_BYTES;
#pragma unroll
                for (int j = 0; j < HD / 16; ++j) {
                    const uint64_t da = desc_k_major(Qs + (j >> 2) * (BM * 128)) + 2 * (j & 3);
                    const uint64_t db = desc_k_major(kt + (j >> 2) * K_CHUNK) + 2 * (j & 3);
                    if (PAIR) umma_bf16_pair(tmem + 128 * (t & 1), da, db, IDESC_QK, j > 0 ? 1u : 0u);
                    else umma_bf16(tmem + 128 * (t & 1), da, db, IDESC_QK, j > 0 ? 1u : 0u);
                }
                commit(&bars->k_empty[t % ST]);
                commit(&bars->s_full[t & 1]);
            };
            if (ok && !mbar_wait(&bars->k_full[0], 0)) { *failed = 3; ok = false; }
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                issue_qk(0);
            }
            for (int t = 0; t < nt && ok; ++t) {
                if (t + 1 < nt) {
                    // the next tile's scores, formed while the softmax warps work on this tile's
                    if (!mbar_wait(&bars->k_full[(t + 1) % ST], ((t + 1) / ST) & 1)) {
                        *failed = 4; ok = false; break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    issue_qk(t + 1);
                }
                if (!mbar_wait(&bars->p_full[t & 1], (t >> 1) & 1) ||
                    !mbar_wait(&bars->v_full[t % ST], (t / ST) & 1)) { *failed = 5; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                // O += P(t) V(t): 8 steps of 16 keys; P from the score tile's first 64 columns
                const unsigned char* vt = Vs + (t % ST) * KV_BYTES;
#pragma unroll
                for (int j = 0; j < BN / 16; ++j) {
                    const uint64_t db = desc_mn_major(vt + j * (16 * 128), V_CHUNK);
                    const uint32_t acc = (t > 0 || j > 0) ? 1u : 0u;
                    if (PAIR) umma_bf16_ts_pair(tmem + O_COL, tmem + 128 * (t & 1) + 8 * j, db, IDESC_PV, acc);
                    else umma_bf16_ts(tmem + O_COL, tmem + 128 * (t & 1) + 8 * j, db, IDESC_PV, acc);
                }
                commit(&bars->v_empty[t % ST]);
                commit(&bars->pv_done);
                if (t == nt - 1) commit(&bars->o_done);
            }
            if (!ok) {   // let nobody wait for what will not come
                commit(&bars->s_full[0]);
                commit(&bars->s_full[1]);
                commit(&bars->pv_done);
                commit(&bars->o_done);
            }
        }
    } else {
        const int quarter = warp & 3;                      // the tensor-memory lanes a warp may touch
        const int half = (warp - 2) >> 2;                  // which 64 keys of a tile, which half of O
        const int row = 32 * quarter + lane;               // tensor-memory lane = query row
        const int head = kvh * G + row / MP;
        const int pos = p0 + row % MP;
        const uint32_t lane_addr = tmem + ((uint32_t)(32 * quarter) << 16);
        // score in units of log 2: c2 * tanh(product * c1) with a cap, product * c1 without
        constexpr float LOG2E = 1.4426950408889634f;
        constexpr float RAISE_BY = 8.0f;
        const bool capped = p.softcap > 0.f;
        const float c1 = capped ? p.scale / p.softcap : p.scale * LOG2E;
        const float c2 = p.softcap * LOG2E;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        // the two threads of a row tell each other a number through shared memory
        auto swap_with_partner = [&](int t, float mine, float& theirs) -> bool {
            xch[((t & 1) * 2 + half) * BM + row] = mine;
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->pair[quarter]);
            if (!mbar_wait(&bars->pair[quarter], t & 1)) return false;
            theirs = xch[((t & 1) * 2 + (half ^ 1)) * BM + row];
            return true;
        };
        for (int t = 0; t < nt && ok; ++t) {
            if (!mbar_wait(&bars->s_full[t & 1], (t >> 1) & 1)) { if (lane == 0) *failed = 6; ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t s_addr = lane_addr + 128 * (t & 1);
            uint32_t raw[64];
            tmem_ld32_issue(s_addr + 64 * half, raw);
            tmem_ld32_issue(s_addr + 64 * half + 32, raw + 32);
            tmem_ld_wait();
            // Which of the thread's 64 keys the row sees: j in [j_lo, j_hi].  A warp whose
            // rows all see all of them takes the path without the mask.
            const int key0 = (kt0 + t) * BN + 64 * half;
            const int j_hi = min(pos, n - 1) - key0;
            const int j_lo = p.window > 0 ? pos - p.window + 1 - key0 : -(1 << 30);
            const bool whole = __all_sync(0xffffffffu, j_lo <= 0 && j_hi >= 63);
            // The row's maximum, taken on the raw products: scaling by a positive factor and
            // the cap are both increasing, so the largest product gives the largest score.
            float mx_raw, other;
            if (whole) mx_raw = row_max<false>(raw, j_lo, j_hi);
            else mx_raw = row_max<true>(raw, j_lo, j_hi);
            if (!swap_with_partner(t, mx_raw, other)) { if (lane == 0) *failed = 9; ok = false; break; }
            mx_raw = fmaxf(mx_raw, other);
            float mx = mx_raw * c1;
            if (capped) mx = c2 * tanh_fast(mx);
            if (mx_raw == -INFINITY) mx = -INFINITY;
            // the reference the exponentials are taken against: raised only by big steps
            float factor = 1.f;
            bool raise = false;
            if (t == 0) {
                m_ref = mx;
            } else if (mx > m_ref + RAISE_BY) {
                raise = true;
                factor = exp2_fast(m_ref - mx);       // 0 when the row had seen no key yet
                m_ref = mx;
            }
            if (__any_sync(0xffffffffu, raise)) {
                // O may be touched once the previous tile's P V has run; each thread of a
                // row rescales its half of the columns
                if (!mbar_wait(&bars->pv_done, (t - 1) & 1)) { if (lane == 0) *failed = 7; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                l *= factor;
#pragma unroll 1
                for (int c = 0; c < HD / 64; ++c) {
                    uint32_t o[32];
                    const uint32_t a = lane_addr + O_COL + (HD / 2) * half + 32 * c;
                    tmem_ld32(a, o);
#pragma unroll
                    for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * factor);
                    tmem_st32(a, o);
                }
            }
            const float ref = m_ref == -INFINITY ? 0.f : m_ref;
            if (capped) {
                if (whole) l += probabilities<true, false>(raw, c1, c2, ref, j_lo, j_hi);
                else l += probabilities<true, true>(raw, c1, c2, ref, j_lo, j_hi);
            } else {
                if (whole) l += probabilities<false, false>(raw, c1, c2, ref, j_lo, j_hi);
                else l += probabilities<false, true>(raw, c1, c2, ref, j_lo, j_hi);
            }
            // P over the first 64 columns of the score tile (both threads have read theirs)
            tmem_st32(s_addr + 32 * half, reinterpret_cast<uint32_t(&)[32]>(raw));
            asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                if (PAIR) mbar_arrive_first_block(&bars->p_full[t & 1]);
                else mbar_arrive(&bars->p_full[t & 1]);
            }
        }
        float l_other = 0.f;
        if (ok && nt > 0) {
            // (pv_done is not waited for tile by tile, so its phase cannot tell the last
            // product from the one before it)
            if (!mbar_wait(&bars->o_done, 0)) { if (lane == 0) *failed = 8; ok = false; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (ok && !swap_with_partner(nt, l, l_other)) { if (lane == 0) *failed = 9; ok = false; }
        }
        // With a split: this warp's rows to `part`, a ticket, and the second to come goes on.
        float w_mine = 1.f, w_theirs = 0.f;
        const float* theirs = nullptr;       // the other half's accumulator columns of this thread
        float l_all = l + l_other;
        if (ok && is_split) {
            // the block's two partial results
            float* mine = p.part + (unit * 2 + part) * part_floats<HD>();
            theirs = p.part + (unit * 2 + (part ^ 1)) * part_floats<HD>();
            // layout: [HD columns][128 rows], then [128 rows][max, sum]
            if (half == 0) {
                mine[(size_t)HD * BM + 2 * row] = m_ref;
                mine[(size_t)HD * BM + 2 * row + 1] = l_all;
            }
#pragma unroll 1
            for (int c = 0; c < HD / 64; ++c) {
                uint32_t o[32];
                const int col0 = (HD / 2) * half + 32 * c;
                tmem_ld32(lane_addr + O_COL + col0, o);
#pragma unroll
                for (int j = 0; j < 32; ++j) mine[(size_t)(col0 + j) * BM + row] = __uint_as_float(o[j]);
            }
            __threadfence();
            __syncwarp();
            int ticket = 0;
            int* counter = p.tickets + unit * 8 + (warp - 2);
            if (lane == 0) ticket = atomicAdd(counter, 1);
            ticket = __shfl_sync(0xffffffffu, ticket, 0);
            if (ticket == 0) {
                ok = false;                   // the other half finishes these rows
            } else {
                __threadfence();
                if (lane == 0) *counter = 0;
                const float m_b = __ldcg(theirs + (size_t)HD * BM + 2 * row);
                const float l_b = __ldcg(theirs + (size_t)HD * BM + 2 * row + 1);
                const float top = fmaxf(m_ref, m_b);
                w_mine = m_ref == -INFINITY ? 0.f : exp2_fast(m_ref - top);
                w_theirs = m_b == -INFINITY ? 0.f : exp2_fast(m_b - top);
                l_all = w_mine * l_all + w_theirs * l_b;
            }
        }
        if (ok) {
            const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
            const bool store = pos < n && pos >= q0;
            __nv_bfloat16* dst = p.out + (size_t)(row0 + pos) * p.n_heads * HD + (size_t)head * HD +
                                 (HD / 2) * half;
#pragma unroll 1
            for (int c = 0; c < HD / 64; ++c) {
                uint32_t o[32];
                const int col0 = (HD / 2) * half + 32 * c;
                tmem_ld32(lane_addr + O_COL + col0, o);
                if (theirs != nullptr) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        o[j] = __float_as_uint(w_mine * __uint_as_float(o[j]) +
                                               w_theirs * __ldcg(theirs + (size_t)(col0 + j) * BM + row));
                }
                if (store) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint32_t w[4];
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            w[k] = pack_bf16(__uint_as_float(o[8 * q4 + 2 * k]) * inv,
                                             __uint_as_float(o[8 * q4 + 2 * k + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + 32 * c + 8 * q4) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (PAIR) cluster_sync_all();     // the other block no longer touches this block's memory or barriers
    if (warp == 1) {
        if (PAIR)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem),
                         "r"(TMEM_COLS)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem),
                         "r"(TMEM_COLS)
                         : "memory");
    }
    if (threadIdx.x == 0 && *failed) atomicExch(p.error_flag, *failed);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn tc_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn) return fn;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
        return nullptr;
    fn = (EncodeTiledFn)ptr;
    return fn;
}

SIB_EXPORT int sib_attention_prefill_tc_supports(int n_heads, int n_kv, int head_dim, int width) {
    if (n_kv <= 0 || n_heads % n_kv) return 0;
    const int G = n_heads / n_kv;
    return (G == 1 || G == 2) && (head_dim == 64 || head_dim == 128 || head_dim == 256) &&
           width % 8 == 0;
}

template <int HD, int G, bool PAIR>
static int launch_tc(const CUtensorMap& map, const TcArgs& p, const TcItems& items, int n_seqs,
                     int max_len, cudaStream_t s) {
    constexpr int ST = (HD == 256 && !PAIR) ? 1 : 2;
    constexpr int NB = PAIR ? 2 : 1;
    const size_t smem = 1024 + (size_t)BM * HD * 2 + 2 * ST * (size_t)BN * HD * 2 / NB + sizeof(Bars) +
                        2 * 2 * BM * sizeof(float) + 16;
    auto kernel = attention_prefill_tc_kernel<HD, G, PAIR>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
        sib_set_error("attention_prefill_tc: shared memory: %s", cudaGetErrorString(e));
        return (int)e;
    }
    constexpr int MP = BM / G;
    const int q_blocks = (max_len + MP - 1) / MP;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(NB * ((q_blocks + NB - 1) / NB), n_seqs, p.n_kv * (p.split_tiles > 0 ? 2 : 1));
    if (items.n > 0) cfg.gridDim = dim3(NB * items.n, 1, 1);
    cfg.blockDim = dim3(320, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    // chained to the kernel before it (see common.cuh), and in clusters of two for pairs
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (sib_chained_launches()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (PAIR) {
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = NB;
        attr[n_attr].val.clusterDim.y = 1;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    e = cudaLaunchKernelEx(&cfg, kernel, map, p, items);
    if (e != cudaSuccess) {
        sib_set_error("attention_prefill_tc: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return sib_check_launch("attention_prefill_tc");
}

// SIB_PREFILL_PAIR=0: one block per 128 query rows also where pairs of blocks could share the tiles.
static bool tc_pairs_allowed() {
    static const bool allowed = [] {
        const char* v = getenv("SIB_PREFILL_PAIR");
        return !(v && v[0] == '0');
    }();
    return allowed;
}

// ---------------------------------------------------------------------------
// BALANCE: the list of work items for prompts whose lengths the host knows.
// ---------------------------------------------------------------------------
namespace {

struct PlanBlock { int b, qblk, nt; };
struct PlanItem { int b, kvh, qblk, part, unit; float cost; };

// What an item costs in units of one key tile: its tiles, what a block pays before its
// first tile and after its last (about 9 us against 2.4 us a tile), and the exchange of a
// split block's partial results.
static float env_float(const char* name, float fallback) {
    const char* v = getenv(name);
    return v ? (float)atof(v) : fallback;
}
static const float ITEM_OVERHEAD = env_float("SIB_PREFILL_ITEM_OVERHEAD", 4.0f);
static const float SPLIT_OVERHEAD = env_float("SIB_PREFILL_SPLIT_OVERHEAD", 1.0f);

// The items when blocks with at least `split_from` key tiles run as two halves; the time
// of the busiest of `slots` places when items are handed out longest first.
float plan_for(const std::vector<PlanBlock>& blocks, int n_kv, int split_from, int slots,
               std::vector<PlanItem>* items, int* n_units) {
    std::vector<PlanItem> list;
    int units = 0;
    for (const PlanBlock& blk : blocks)
        for (int kvh = 0; kvh < n_kv; ++kvh) {
            if (blk.nt >= split_from && blk.nt >= 2) {
                const int first_half = (blk.nt + 1) / 2;
                list.push_back({blk.b, kvh, blk.qblk, 0, units, first_half + ITEM_OVERHEAD + SPLIT_OVERHEAD});
                list.push_back({blk.b, kvh, blk.qblk, 1, units,
                                blk.nt - first_half + ITEM_OVERHEAD + SPLIT_OVERHEAD});
                ++units;
            } else {
                list.push_back({blk.b, kvh, blk.qblk, 0, -1, blk.nt + ITEM_OVERHEAD});
            }
        }
    std::stable_sort(list.begin(), list.end(),
                     [](const PlanItem& x, const PlanItem& y) { return x.cost > y.cost; });
    std::priority_queue<float, std::vector<float>, std::greater<float>> busy;
    for (int i = 0; i < slots; ++i) busy.push(0.f);
    float longest = 0.f;
    for (const PlanItem& it : list) {
        const float t = busy.top() + it.cost;
        busy.pop();
        busy.push(t);
        longest = std::max(longest, t);
    }
    if (items) *items = list;
    if (n_units) *n_units = units;
    return longest;
}

bool plan_items_now(const int* lens, const int* q0s, int n_seqs, int n_kv, int G, int head_dim,
                    int window, int sms, TcItems* out, int* n_units);

// Fills `out` for prompts of `lens` (host memory); false if a list does not fit or pay.
// (Every layer of a step asks for the same few plans: the last ones are kept.)
bool plan_items(const int* lens, const int* q0s, int n_seqs, int n_kv, int G, int head_dim,
                int window, int sms, TcItems* out, int* n_units) {
    struct Kept {
        std::vector<int> key;
        TcItems items;
        int units = 0;
        bool ok = false;
    };
    static thread_local Kept kept[4];
    static thread_local int next = 0;
    if (!lens || n_seqs <= 0) return false;
    std::vector<int> key(lens, lens + n_seqs);
    for (int b = 0; b < n_seqs; ++b) key.push_back(q0s ? q0s[b] : 0);
    const int tail[6] = {n_kv, G, head_dim, window, sms, tc_pairs_allowed() ? 1 : 0};
    key.insert(key.end(), tail, tail + 6);
    for (Kept& k : kept)
        if (k.key == key) {
            if (k.ok) {
                *out = k.items;
                if (n_units) *n_units = k.units;
            }
            return k.ok;
        }
    Kept& k = kept[next];
    next = (next + 1) % 4;
    k.key = key;
    k.units = 0;
    k.ok = plan_items_now(lens, q0s, n_seqs, n_kv, G, head_dim, window, sms, &k.items, &k.units);
    if (k.ok) {
        *out = k.items;
        if (n_units) *n_units = k.units;
    }
    return k.ok;
}

bool plan_items_now(const int* lens, const int* q0s, int n_seqs, int n_kv, int G, int head_dim,
                    int window, int sms, TcItems* out, int* n_units) {
    static const bool allowed = [] {
        const char* v = getenv("SIB_PREFILL_BALANCE");
        return !(v && v[0] == '0');
    }();
    if (!allowed || !lens || n_seqs <= 0 || n_seqs >= 4096 || n_kv > 255) return false;
    const bool pair = head_dim >= 128 && tc_pairs_allowed();
    const int NB = pair ? 2 : 1, span = NB * (BM / G), slots = std::max(1, sms / NB);
    std::vector<PlanBlock> blocks;
    int nt_max = 0;
    for (int b = 0; b < n_seqs; ++b) {
        const int n = lens[b];
        if (n < 0) return false;
        // (blocks of rows that are keys only have no work)
        for (int q = (q0s ? std::max(0, q0s[b]) : 0) / span; q * span < n; ++q) {
            if (q >= 4096 || (long long)(blocks.size() + 1) * n_kv > MAX_ITEMS) return false;
            const int first0 = q * span, k_hi = std::min(n, first0 + span);
            const int k_lo = window > 0 ? std::max(0, first0 - window + 1) : 0;
            const int nt = (k_hi + BN - 1) / BN - k_lo / BN;
            blocks.push_back({b, q, nt});
            nt_max = std::max(nt_max, nt);
        }
    }
    if (blocks.empty()) return false;
    // no split, or every block from some length on
    int best_from = nt_max + 1;
    float best = plan_for(blocks, n_kv, best_from, slots, nullptr, nullptr);
    for (int from = nt_max; from >= 2; --from) {
        long long count = 0;
        for (const PlanBlock& blk : blocks) count += (blk.nt >= from ? 2 : 1) * n_kv;
        if (count > MAX_ITEMS) break;
        const float t = plan_for(blocks, n_kv, from, slots, nullptr, nullptr);
        if (t < best - 0.25f) {
            best = t;
            best_from = from;
        }
    }
    std::vector<PlanItem> items;
    plan_for(blocks, n_kv, best_from, slots, &items, n_units);
    out->n = (int)items.size();
    for (size_t i = 0; i < items.size(); ++i) {
        const PlanItem& it = items[i];
        out->where[i] = ((uint32_t)it.b << 20) | ((uint32_t)it.kvh << 12) | (uint32_t)it.qblk;
        out->what[i] = (it.unit < 0 ? 0xFFFFFFu : (uint32_t)it.unit) | ((uint32_t)it.part << 24);
    }
    return true;
}

int device_sms() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return 0;
    return sms;
}

}  // namespace

// What a launch for prompts of these lengths (host memory) needs to run as a balanced list
// of work items: bytes of scratch memory and ticket counters (int, zero between launches)
// for the blocks it splits.  Returns the number of items, 0 if such a launch is a grid.
SIB_EXPORT int sib_attention_prefill_tc_plan(const int* host_lens, const int* host_q0, int n_seqs,
                                             int n_heads, int n_kv, int head_dim, int window,
                                             long long* scratch_bytes, int* n_tickets) {
    if (scratch_bytes) *scratch_bytes = 0;
    if (n_tickets) *n_tickets = 0;
    if (n_kv <= 0 || n_heads % n_kv) return 0;
    TcItems items;
    int units = 0;
    if (!plan_items(host_lens, host_q0, n_seqs, n_kv, n_heads / n_kv, head_dim, window, device_sms(),
                    &items, &units))
        return 0;
    const int nb = (head_dim >= 128 && tc_pairs_allowed()) ? 2 : 1;
    if (scratch_bytes)
        *scratch_bytes = (long long)units * nb * 2 * (long long)BM * (head_dim + 2) * sizeof(float);
    if (n_tickets) *n_tickets = units * nb * 8;
    return items.n;
}

// Attention of `n_seqs` packed prompts that all start at position 0; `total_rows`
// is the number of rows of the packed buffer.  `seq_q0` (device; `host_q0` the same on the
// host, for the planner; both null: none): the rows of a sequence before this position
// bring keys and values only, their output rows are not written (a step that continues
// sequences puts what they hold there, see sib_gather_kv_rows).
// Whether a launch of this shape would split its long blocks of query rows (see SPLIT at the
// top): it does when its blocks would fill at most half of the device.  Returns
// the number of key tiles from which a block is split (0: no split) and what the launch then
// needs: bytes of scratch memory and ticket counters (int, zero between launches).
SIB_EXPORT int sib_attention_prefill_tc_split(int n_seqs, int max_len, int n_heads, int n_kv,
                                              int head_dim, long long* scratch_bytes,
                                              int* n_tickets) {
    if (scratch_bytes) *scratch_bytes = 0;
    if (n_tickets) *n_tickets = 0;
    if (n_kv <= 0 || n_heads % n_kv || n_seqs <= 0 || max_len <= 0) return 0;
    static const bool allowed = [] {
        const char* v = getenv("SIB_PREFILL_SPLIT");
        return !(v && v[0] == '0');
    }();
    if (!allowed) return 0;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return 0;
    const int G = n_heads / n_kv, MP = BM / G;
    const bool pair = head_dim >= 128 && tc_pairs_allowed();
    const int nb = pair ? 2 : 1;
    const long long q_blocks = nb * (((max_len + MP - 1) / MP + nb - 1) / nb);
    const long long blocks = q_blocks * n_seqs * n_kv;
    // (measured: a split that pushes the launch into a second wave of blocks loses more than
    // it gains, since every block pays about 9 us of start-up before its first tile)
    if (2 * blocks > sms) return 0;
    if (scratch_bytes) *scratch_bytes = blocks * 2 * (long long)BM * (head_dim + 2) * sizeof(float);
    if (n_tickets) *n_tickets = (int)(blocks * 8);
    return 6;
}

SIB_EXPORT int sib_attention_prefill_tc(const void* qkv, int width, int total_rows, void* out,
                                        const int* seq_row0, const int* seq_len, int n_seqs,
                                        int max_len, int n_heads, int n_kv, int head_dim,
                                        float scale, float softcap, int window, void* scratch,
                                        long long scratch_bytes, int* tickets, int n_tickets,
                                        const int* host_lens, const int* seq_q0, const int* host_q0,
                                        void* stream) {
    if (n_seqs == 0 || max_len == 0) return 0;
    SIB_REQUIRE(sib_attention_prefill_tc_supports(n_heads, n_kv, head_dim, width),
                "attention_prefill_tc: heads=%d kv_heads=%d head_dim=%d is not a shape this kernel "
                "takes (1 or 2 heads per kv head; head_dim 64, 128 or 256)", n_heads, n_kv, head_dim);
    SIB_REQUIRE(width == (n_heads + 2 * n_kv) * head_dim && ((uintptr_t)qkv % 16) == 0 &&
                    ((uintptr_t)out % 16) == 0 && total_rows > 0,
                "attention_prefill_tc: packed rows of %d elements do not fit the head counts", width);
    SIB_REQUIRE(n_seqs > 0 && n_seqs < 65536 && n_kv < 65536 && max_len > 0 && window >= 0,
                "attention_prefill_tc: seqs=%d max_len=%d", n_seqs, max_len);
    // the row maximum is taken before scaling, which holds for a positive factor only
    SIB_REQUIRE(scale > 0.f && softcap >= 0.f, "attention_prefill_tc: score scale %g and cap %g "
                "must be positive (cap 0: none)", (double)scale, (double)softcap);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    SIB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, "attention_prefill_tc: no current device");
    int* error_flag = sib_error_word(SIB_ERR_ATTENTION_PREFILL_TC);
    if (!error_flag) return -1;
    EncodeTiledFn enc = tc_encode_fn();
    SIB_REQUIRE(enc != nullptr, "attention_prefill_tc: cuTensorMapEncodeTiled is not available");
    CUtensorMap map;
    cuuint64_t dims[2] = {(cuuint64_t)width, (cuuint64_t)total_rows};
    cuuint64_t strides[1] = {(cuuint64_t)width * 2};
    cuuint32_t box[2] = {64, 64};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(qkv), dims, strides,
                     box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    SIB_REQUIRE(r == CUDA_SUCCESS, "attention_prefill_tc: cuTensorMapEncodeTiled failed with code %d",
                (int)r);
    // long blocks are split if the caller brought the memory for it
    long long need_bytes = 0;
    int need_tickets = 0;
    int split_tiles = sib_attention_prefill_tc_split(n_seqs, max_len, n_heads, n_kv, head_dim,
                                                     &need_bytes, &need_tickets);
    if (scratch == nullptr || tickets == nullptr || scratch_bytes < need_bytes ||
        n_tickets < need_tickets || ((uintptr_t)scratch % 16) != 0)
        split_tiles = 0;
    const int G = n_heads / n_kv;
    // with the lengths known on the host: a balanced list of work items, if the caller
    // brought the memory that its split blocks need
    static thread_local TcItems items;
    items.n = 0;
    if (host_lens) {
        int units = 0;
        if (plan_items(host_lens, host_q0, n_seqs, n_kv, G, head_dim, window, device_sms(), &items,
                       &units)) {
            const int nb = (head_dim >= 128 && tc_pairs_allowed()) ? 2 : 1;
            const long long bytes = (long long)units * nb * 2 * (long long)BM * (head_dim + 2) * sizeof(float);
            if (units > 0 && (scratch == nullptr || tickets == nullptr || scratch_bytes < bytes ||
                              n_tickets < units * nb * 8 || ((uintptr_t)scratch % 16) != 0))
                items.n = 0;
        } else {
            items.n = 0;
        }
    }
    if (items.n > 0) split_tiles = 0;
    TcArgs p{(__nv_bfloat16*)out, seq_row0, seq_len, seq_q0, error_flag, (float*)scratch, tickets,
             split_tiles, n_heads, n_kv, window, scale, softcap};
    cudaStream_t s = (cudaStream_t)stream;
#define BY_G(HD, PAIR)                                                         \
    do {                                                                       \
        if (G == 1) return launch_tc<HD, 1, PAIR>(map, p, items, n_seqs, max_len, s); \
        return launch_tc<HD, 2, PAIR>(map, p, items, n_seqs, max_len, s);             \
    } while (0)
    if (head_dim == 64) BY_G(64, false);
    if (tc_pairs_allowed()) {
        if (head_dim == 128) BY_G(128, true);
        BY_G(256, true);
    }
    if (head_dim == 128) BY_G(128, false);
    BY_G(256, false);
#undef BY_G
}
