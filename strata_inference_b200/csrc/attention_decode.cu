// Attention of single query rows over the paged bfloat16 cache: the
// bandwidth-bound kernel of decoding.  Same mathematics as attention_rows.cu
// (scale, soft cap, causal and window mask, softmax in 32-bit, weighted sum of
// v); this file only changes how the work is laid out:
//
// * one block of 1, 2, 4 or 8 warps per (row, kv head, split), each warp an equal
//   share of the split's keys: the G = n_heads / n_kv query heads that share a kv
//   head are done together, so each key and value is read once;
// * keys are walked in tiles of 16 positions, aligned so that a tile lies in
//   one page.  Scores of a tile are one mma.m16n8k16 chain: the 16 keys are the
//   A operand, the (up to 8) query heads the B operand, fragments loaded
//   straight from global memory with 16-byte loads under the same permutation of
//   the head dimension on both operands (see linear_skinny.cu);
// * probabilities go through a few hundred bytes of shared memory per warp; the
//   weighted sum of v runs on the CUDA cores with each lane owning 8 consecutive
//   dimensions of a value row (a 16-byte load), several keys per pass when the
//   head is narrower than 256;
// * the warps' partial (max, sum, accumulator) are joined in shared memory.  With
//   splits > 1 the block's partial goes to scratch memory and the block takes a
//   ticket of its (row, kv head); the block that draws the last ticket joins all
//   the splits and writes the output, so no second kernel is needed.  The ticket
//   counters are zero between launches: the last block puts its counter back.
//   Neither join has a loop of one thread or a barrier of its own where the sizes
//   allow it: every thread makes the warps' weights for its columns itself, and the
//   last block's warps join their own columns (join_runs_by_warp).
//
// Plain counterpart: tests/plain_gemma2.py attention().
// Reference: src/backend/cuda/kernels.rs:2851-3180 (grouped_attn_decode: one block
// per head, two passes over the keys), src/backend/cpu.rs:1352-1434.
#include "common.cuh"

struct AttnDecodeArgs {
    const __nv_bfloat16* q;   // row r, head h at q + r * q_stride + h * head_dim
    const __nv_bfloat16* k_pool;
    const __nv_bfloat16* v_pool;
    __nv_bfloat16* out;       // [rows, n_heads * head_dim]
    float* partial;           // [rows, n_heads, splits, head_dim + 2]
    int* tickets;             // [rows, n_kv], zero between launches
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* page_table;
    int q_stride;
    int rows, n_heads, n_kv;
    int max_pages, page_tokens, ring_tokens;
    int window, splits;
    float scale, softcap;
    // The kernel before this one wrote at most the last `fresh` positions of a row's sequence
    // (1 in a single-token step): tiles of keys below them may be loaded before that kernel
    // has finished.  0: every load waits for it.
    int fresh;
};

__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ld_stream16(const __nv_bfloat16* p) {
    uint4 v;
    asm("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
        : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
        : "l"(p));
    return v;
}

__device__ __forceinline__ void unpack8(const uint4& v, float (&o)[8]) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        o[2 * i] = __uint_as_float(w[i] << 16);
        o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// The most splits of a (row, kv head) a launch takes.
constexpr int MAX_SPLITS = 128;

// The join of the runs of a (row, kv head) by the block that drew the last ticket, without a
// barrier: a thread takes NITEM pairs of output columns (pair threadIdx.x, then threadIdx.x +
// blockDim.x; all lanes of a warp work on one head, since HD / 2 is a multiple of 32) and a
// lane the maximum and the sum of run `lane` (and lane + 32 with NRUN 64).  Every
// accumulator that a thread needs and its lane's runs' maxima and sums are asked for at
// once, one round trip; the runs' weights are made with the warp's shuffles.  For at most
// NRUN runs and G * HD / 2 <= NITEM * blockDim.x.
template <int HD, int G, int NITEM, int NRUN>
__device__ __forceinline__ void join_runs_by_warp(const float* unit_partial, int splits,
                                                  __nv_bfloat16* out_row, int lane) {
    constexpr int PW = HD + 2;
    constexpr int LR = (NRUN + 31) / 32;     // runs a lane answers for
    float2 v[NITEM][NRUN], ml[NITEM][LR];
#pragma unroll
    for (int k = 0; k < NITEM; ++k) {
        const int item = threadIdx.x + k * blockDim.x;
        const bool live = item < G * HD / 2;                  // (the same for a whole warp)
        const int h = live ? item / (HD / 2) : 0, d = 2 * (item % (HD / 2));
        const float* ph = unit_partial + (size_t)h * splits * PW;
#pragma unroll
        for (int b = 0; b < NRUN; ++b)
            v[k][b] = live && b < splits
                          ? __ldcg(reinterpret_cast<const float2*>(ph + (size_t)b * PW + 2 + d))
                          : make_float2(0.f, 0.f);
#pragma unroll
        for (int j = 0; j < LR; ++j)
            ml[k][j] = live && lane + 32 * j < splits
                           ? __ldcg(reinterpret_cast<const float2*>(ph + (size_t)(lane + 32 * j) * PW))
                           : make_float2(-INFINITY, 0.f);
    }
#pragma unroll
    for (int k = 0; k < NITEM; ++k) {
        const int item = threadIdx.x + k * blockDim.x;
        if (item >= G * HD / 2) continue;
        const int h = item / (HD / 2), d = 2 * (item % (HD / 2));
        float mx = ml[k][0].x;
#pragma unroll
        for (int j = 1; j < LR; ++j) mx = fmaxf(mx, ml[k][j].x);
        mx = warp_max(mx);
        float f[LR], part = 0.f;
#pragma unroll
        for (int j = 0; j < LR; ++j) {
            f[j] = ml[k][j].x == -INFINITY ? 0.f : expf(ml[k][j].x - mx);   // a run without keys
            part += f[j] * ml[k][j].y;
        }
        const float sum = warp_sum(part);
        float2 a = make_float2(0.f, 0.f);
#pragma unroll
        for (int b = 0; b < NRUN; ++b) {         // in run order; runs beyond the last weigh 0
            const float fb = __shfl_sync(0xffffffffu, f[b / 32], b % 32);
            a.x += fb * v[k][b].x;
            a.y += fb * v[k][b].y;
        }
        const float inv = 1.0f / sum;
        *reinterpret_cast<__nv_bfloat162*>(out_row + h * HD + d) =
            __floats2bfloat162_rn(a.x * inv, a.y * inv);
    }
}

// HD: head size (64, 128 or 256).  G: query heads per kv head (1, 2, 4 or 8).  EARLY: the first
// tile of keys may be fetched before the kernel ahead of this one has finished (it shortens
// the chain of waits of a step of one row: batch 1 runs 1.5 % faster with it; with more rows
// the registers that the tile holds across the wait cost more than the wait: batch 2 ran 3 %
// and batch 8 2 % slower with it).
// WIDE: blocks of 8 warps (a single row's step: half as many partial results to join as with
// blocks of 4); the narrower kernel keeps its registers and shared memory as they were.
template <int HD, int G, bool EARLY, bool WIDE = false>
__global__ void __launch_bounds__(WIDE ? 256 : 128) attention_decode_kernel(AttnDecodeArgs p) {
    constexpr int KB = HD / 32;          // 32-wide blocks of the head dimension
    constexpr int LPK = HD / 8;          // lanes that cover one value row
    constexpr int KPP = 32 / LPK;        // keys per pass of the weighted sum
    constexpr int PW = HD + 2;           // a partial: max, sum, HD accumulators
    __shared__ float sm_all[WIDE ? 8 : 4][2][16][8];
    extern __shared__ __align__(16) float part_dyn[];          // [warps][G][PW]
    float(*part_sm)[G][PW] = reinterpret_cast<float(*)[G][PW]>(part_dyn);
    __shared__ float w_sm[G][MAX_SPLITS];
    __shared__ float l_sm[G][MAX_SPLITS];
    __shared__ float ml_sm[G][2];
    __shared__ int ticket_sm;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    float(*s_sm)[8] = sm_all[warp][0];
    float(*p_sm)[8] = sm_all[warp][1];
    pdl_trigger();
    const int split = (int)(blockIdx.x % p.splits);
    const int kvh = (int)((blockIdx.x / p.splits) % p.n_kv);
    const int r = (int)(blockIdx.x / ((unsigned)p.splits * p.n_kv));
    const int g = lane >> 2, t = lane & 3;

    // Where the row is and which pages it reads: written by the host before the step, not
    // by the kernel before this one, so this chain of dependent loads need not wait for it.
    const int pos = p.row_pos[r];
    const int slot = p.seq_slot[p.row_seq[r]];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int tile_lo = lo >> 4, tile_hi = pos >> 4;             // inclusive
    const int n_tiles = tile_hi - tile_lo + 1;
    const int per = (n_tiles + nw * p.splits - 1) / (nw * p.splits);
    const int t0 = tile_lo + (split * nw + warp) * per;
    const int t1 = min(t0 + per, tile_hi + 1);
    const int* table = p.page_table + (size_t)slot * p.max_pages;
    if (t0 < t1) {
        const int cell0 = p.ring_tokens > 0 ? (t0 << 4) % p.ring_tokens : (t0 << 4);
        asm volatile("prefetch.global.L1 [%0];\n" ::"l"(table + cell0 / p.page_tokens));
    }
    // One tile of keys and values: every load is issued before anything waits on one.
    uint4 ka_r[KB], kb_r[KB], v_r[16 / KPP];
    const int sub = lane / LPK;          // which key of a pass this lane works on
    const int dim0 = (lane % LPK) * 8;   // its 8 dimensions
    auto load_tile = [&](int tile) {
        const int base = tile << 4;
        const int cell = p.ring_tokens > 0 ? base % p.ring_tokens : base;
        const int page = table[cell / p.page_tokens];
        const size_t tile_off =
            (((size_t)page * p.n_kv + kvh) * p.page_tokens + cell % p.page_tokens) * HD;
        const __nv_bfloat16* kt = p.k_pool + tile_off;
        const __nv_bfloat16* vt = p.v_pool + tile_off;
        const int last = pos - base;                              // keys beyond `last` do not exist
        const int ka = min(g, last), kb2 = min(g + 8, last);      // clamped: loads stay in the sequence
#pragma unroll
        for (int j = 0; j < KB; ++j) {
            ka_r[j] = ld_stream16(kt + (size_t)ka * HD + 32 * j + 8 * t);
            kb_r[j] = ld_stream16(kt + (size_t)kb2 * HD + 32 * j + 8 * t);
        }
#pragma unroll
        for (int i = 0; i < 16 / KPP; ++i)
            v_r[i] = ld_stream16(vt + (size_t)min(i * KPP + sub, last) * HD + dim0);
    };
    // the first tile's keys and values, if the kernel before this one cannot have written them
    const bool early = EARLY && p.fresh > 0 && t0 < t1 && (t0 << 4) + 15 < pos - p.fresh + 1;
    if (early) load_tile(t0);
    pdl_wait();

    // query heads of this kv head as the B operand: lane (g, t) holds head g
    uint4 qf[KB];
    {
        const __nv_bfloat16* qp = p.q + (size_t)r * p.q_stride + (size_t)(kvh * G + g) * HD;
#pragma unroll
        for (int j = 0; j < KB; ++j)
            qf[j] = g < G ? __ldg(reinterpret_cast<const uint4*>(qp + 32 * j + 8 * t))
                          : make_uint4(0, 0, 0, 0);
    }

    float m[G], l[G], acc[G][8];
#pragma unroll
    for (int h = 0; h < G; ++h) {
        m[h] = -INFINITY;
        l[h] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[h][e] = 0.f;
    }

    for (int tile = t0; tile < t1; ++tile) {
        const int base = tile << 4;                               // first position of the tile
        if (!(early && tile == t0)) load_tile(tile);
        // ---- scores: 16 keys x G heads ----
        float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < KB; ++j) {
            mma16816(c, ka_r[j].x, kb_r[j].x, ka_r[j].y, kb_r[j].y, qf[j].x, qf[j].y);
            mma16816(c, ka_r[j].z, kb_r[j].z, ka_r[j].w, kb_r[j].w, qf[j].z, qf[j].w);
        }
        // c[0], c[1]: key g, heads 2t, 2t+1;  c[2], c[3]: key g + 8
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = g + (i >= 2 ? 8 : 0), head = 2 * t + (i & 1);
            if (head < G) {
                float s = c[i] * p.scale;
                if (p.softcap > 0.f) s = p.softcap * tanhf(s / p.softcap);
                const int kpos = base + key;
                s_sm[key][head] = (kpos >= lo && kpos <= pos) ? s : -INFINITY;
            }
        }
        __syncwarp();
        float corr[G];
#pragma unroll
        for (int h = 0; h < G; ++h) {
            float mx = m[h];
#pragma unroll
            for (int key = 0; key < 16; ++key) mx = fmaxf(mx, s_sm[key][h]);
            corr[h] = expf(m[h] - mx);
            m[h] = mx;
            l[h] *= corr[h];
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[h][e] *= corr[h];
        }
        if (lane < 16) {
#pragma unroll
            for (int h = 0; h < G; ++h) p_sm[lane][h] = expf(s_sm[lane][h] - m[h]);
        }
        __syncwarp();
        // ---- weighted sum of v: KPP keys per pass, 8 dimensions per lane ----
#pragma unroll
        for (int k0 = 0; k0 < 16; k0 += KPP) {
            const int key = k0 + sub;
            float vf[8];
            unpack8(v_r[k0 / KPP], vf);
#pragma unroll
            for (int h = 0; h < G; ++h) {
                const float w = p_sm[key][h];
#pragma unroll
                for (int e = 0; e < 8; ++e) acc[h][e] += w * vf[e];
            }
        }
#pragma unroll
        for (int h = 0; h < G; ++h) {
#pragma unroll
            for (int key = 0; key < 16; ++key) l[h] += p_sm[key][h];
        }
        __syncwarp();
    }

    // lanes that worked on different keys of a pass hold partial sums of the same dimensions
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
#pragma unroll
        for (int h = 0; h < G; ++h)
#pragma unroll
            for (int e = 0; e < 8; ++e) acc[h][e] += __shfl_xor_sync(0xffffffffu, acc[h][e], o);
    }
    // ---- the warps' partials joined in shared memory ----
    if (sub == 0) {
#pragma unroll
        for (int h = 0; h < G; ++h) {
            if (lane == 0) { part_sm[warp][h][0] = m[h]; part_sm[warp][h][1] = l[h]; }
#pragma unroll
            for (int e = 0; e < 8; ++e) part_sm[warp][h][2 + dim0 + e] = acc[h][e];
        }
    }
    __syncthreads();
    __nv_bfloat16* out_row = p.out + (size_t)r * p.n_heads * HD + (size_t)kvh * G * HD;
    float* my_partial = p.partial + (((size_t)r * p.n_heads + kvh * G) * p.splits + split) * PW;
    // (every thread makes the warps' weights for its head itself: no thread's loop and no
    // second barrier between the warps' results and their sum)
    for (int item = threadIdx.x; item < G * HD / 2; item += blockDim.x) {
        const int h = item / (HD / 2), d = 2 * (item % (HD / 2));
        float mx = -INFINITY;
        for (int w = 0; w < nw; ++w) mx = fmaxf(mx, part_sm[w][h][0]);
        float sum = 0.f;
        float2 a = make_float2(0.f, 0.f);
        for (int w = 0; w < nw; ++w) {                      // in warp order
            const float mw = part_sm[w][h][0];
            const float f = mw == -INFINITY ? 0.f : expf(mw - mx);   // a warp without keys
            sum += f * part_sm[w][h][1];
            const float2 v = *reinterpret_cast<const float2*>(&part_sm[w][h][2 + d]);
            a.x += f * v.x;
            a.y += f * v.y;
        }
        if (p.splits == 1) {
            const float inv = 1.0f / sum;
            *reinterpret_cast<__nv_bfloat162*>(out_row + h * HD + d) =
                __floats2bfloat162_rn(a.x * inv, a.y * inv);
        } else {
            float* pp = my_partial + (size_t)h * p.splits * PW;
            if (d == 0) *reinterpret_cast<float2*>(pp) = make_float2(mx, sum);
            *reinterpret_cast<float2*>(pp + 2 + d) = a;
        }
    }
    if (p.splits == 1) return;

    // ---- the block that finishes last joins the splits ----
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) ticket_sm = atomicAdd(p.tickets + r * p.n_kv + kvh, 1);
    __syncthreads();
    if (ticket_sm != p.splits - 1) return;
    __threadfence();
    const float* unit_partial = p.partial + ((size_t)r * p.n_heads + kvh * G) * p.splits * PW;
    // Few enough runs and columns for a warp to join its columns by itself (before: maxima, a
    // barrier, one thread's loop over the runs, a barrier, the sums' loads, a barrier, a loop,
    // a barrier, then the accumulators).
    {
        constexpr int ITEMS = G * HD / 2;
        bool joined = true;
        if (WIDE && ITEMS <= 256 && p.splits <= 32)
            join_runs_by_warp<HD, G, 1, 32>(unit_partial, p.splits, out_row, lane);
        else if (WIDE && ITEMS <= 256 && p.splits <= 64)
            join_runs_by_warp<HD, G, 1, 64>(unit_partial, p.splits, out_row, lane);
        else if (WIDE && ITEMS <= 512 && p.splits <= 32)
            join_runs_by_warp<HD, G, 2, 32>(unit_partial, p.splits, out_row, lane);
        else if (!WIDE && ITEMS <= (int)blockDim.x && p.splits <= 32)
            join_runs_by_warp<HD, G, 1, 32>(unit_partial, p.splits, out_row, lane);
        else if (!WIDE && ITEMS <= 2 * (int)blockDim.x && p.splits <= 16)
            join_runs_by_warp<HD, G, 2, 16>(unit_partial, p.splits, out_row, lane);
        else if (!WIDE && HD == 256 && ITEMS <= 2 * (int)blockDim.x && p.splits <= 32) {
            // (only where the loop over the keys needs as many registers anyway: at smaller
            // head sizes this would cost a resident block)
            if constexpr (HD == 256)
                join_runs_by_warp<HD, G, 2, 32>(unit_partial, p.splits, out_row, lane);
        }
        else
            joined = false;
        if (joined) {
            if (threadIdx.x == 0) p.tickets[r * p.n_kv + kvh] = 0;
            return;
        }
    }
    for (int i = threadIdx.x; i < G * p.splits; i += blockDim.x)
        w_sm[i / p.splits][i % p.splits] = __ldcg(unit_partial + (size_t)i * PW);       // the maxima
    __syncthreads();
    if (threadIdx.x < G) {
        const int h = threadIdx.x;
        float mx = -INFINITY;
        for (int b = 0; b < p.splits; ++b) mx = fmaxf(mx, w_sm[h][b]);
        ml_sm[h][0] = mx;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < G * p.splits; i += blockDim.x) {
        const int h = i / p.splits, b = i % p.splits;
        const float mb = w_sm[h][b];
        const float f = mb == -INFINITY ? 0.f : expf(mb - ml_sm[h][0]);
        w_sm[h][b] = f;
        l_sm[h][b] = f * __ldcg(unit_partial + (size_t)i * PW + 1);
    }
    __syncthreads();
    if (threadIdx.x < G) {
        const int h = threadIdx.x;
        float sum = 0.f;
        for (int b = 0; b < p.splits; ++b) sum += l_sm[h][b];        // in run order
        ml_sm[h][1] = sum;
    }
    __syncthreads();
    // the weighted sum of the runs' accumulators, 8 loads in flight per thread
    for (int item = threadIdx.x; item < G * HD / 2; item += blockDim.x) {
        const int h = item / (HD / 2), d = 2 * (item % (HD / 2));
        const float* pp = unit_partial + (size_t)h * p.splits * PW + 2 + d;
        float2 a = make_float2(0.f, 0.f);
        int b = 0;
        for (; b + 8 <= p.splits; b += 8) {
            float2 v[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                v[u] = __ldcg(reinterpret_cast<const float2*>(pp + (size_t)(b + u) * PW));
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                const float f = w_sm[h][b + u];
                a.x += f * v[u].x;
                a.y += f * v[u].y;
            }
        }
        for (; b < p.splits; ++b) {
            const float f = w_sm[h][b];
            const float2 v = __ldcg(reinterpret_cast<const float2*>(pp + (size_t)b * PW));
            a.x += f * v.x;
            a.y += f * v.y;
        }
        const float inv = 1.0f / ml_sm[h][1];
        *reinterpret_cast<__nv_bfloat162*>(out_row + h * HD + d) =
            __floats2bfloat162_rn(a.x * inv, a.y * inv);
    }
    if (threadIdx.x == 0) p.tickets[r * p.n_kv + kvh] = 0;
}

// 1 if this kernel takes the shape (else the caller uses attention_rows).
SIB_EXPORT int sib_attention_decode_supports(int n_heads, int n_kv, int head_dim, int page_tokens) {
    if (n_kv <= 0 || n_heads % n_kv) return 0;
    const int G = n_heads / n_kv;
    const bool g_ok = G == 1 || G == 2 || G == 4 || G == 8;
    const bool hd_ok = head_dim == 64 || head_dim == 128 || head_dim == 256;
    return g_ok && hd_ok && page_tokens % 16 == 0;
}

// How many warps of this kernel the current device holds at a time for the shape (blocks of
// 4 warps that fit on an SM, by the kernel's registers and shared memory, times the SMs):
// what a caller sizes its split of the keys by.  0 if the shape is not one this kernel takes.
static int resident_warps(int n_heads, int n_kv, int head_dim, int warps);

SIB_EXPORT int sib_attention_decode_resident_warps(int n_heads, int n_kv, int head_dim) {
    return resident_warps(n_heads, n_kv, head_dim, 4);
}

// The same for blocks of `warps` warps (8: the wide kernel, which has room for fewer blocks).
SIB_EXPORT int sib_attention_decode_resident_warps_of(int n_heads, int n_kv, int head_dim, int warps) {
    if (warps != 1 && warps != 2 && warps != 4 && warps != 8) return 0;
    return resident_warps(n_heads, n_kv, head_dim, warps);
}

static int resident_warps(int n_heads, int n_kv, int head_dim, int warps) {
    if (!sib_attention_decode_supports(n_heads, n_kv, head_dim, 16)) return 0;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
        return 0;
    const int G = n_heads / n_kv;
    int per_sm = 0;
    cudaError_t e = cudaErrorInvalidValue;
#define ASK(HD, GG)                                                                         \
    if (warps == 8 && (size_t)8 * GG * (HD + 2) * sizeof(float) > 32 * 1024)                \
        cudaFuncSetAttribute(attention_decode_kernel<HD, GG, false, true>,                  \
                             cudaFuncAttributeMaxDynamicSharedMemorySize,                   \
                             (int)((size_t)8 * GG * (HD + 2) * sizeof(float)));             \
    e = warps == 8                                                                          \
            ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(                                \
                  &per_sm, attention_decode_kernel<HD, GG, false, true>, 256,               \
                  (size_t)8 * GG * (HD + 2) * sizeof(float))                                \
            : cudaOccupancyMaxActiveBlocksPerMultiprocessor(                                \
                  &per_sm, attention_decode_kernel<HD, GG, false>, 32 * warps,              \
                  (size_t)warps * GG * (HD + 2) * sizeof(float))
#define BY_G(HD)                    \
    do {                            \
        if (G == 1) { ASK(HD, 1); }      \
        else if (G == 2) { ASK(HD, 2); } \
        else if (G == 4) { ASK(HD, 4); } \
        else { ASK(HD, 8); }             \
    } while (0)
    if (head_dim == 64) BY_G(64);
    else if (head_dim == 128) BY_G(128);
    else BY_G(256);
#undef BY_G
#undef ASK
    if (e != cudaSuccess || per_sm <= 0) return 0;
    return per_sm * warps * sms;
}

static int attention_decode(
    const void* q, int q_stride, const void* k_pool, const void* v_pool, const int* page_table,
    int max_pages, int page_tokens, int ring_tokens, const int* row_pos, const int* row_seq,
    const int* seq_slot, void* out, float* partial, int* tickets, int rows, int n_heads, int n_kv,
    int head_dim, float scale, float softcap, int window, int splits, int warps, int fresh,
    void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(sib_attention_decode_supports(n_heads, n_kv, head_dim, page_tokens),
                "attention_decode: heads=%d kv_heads=%d head_dim=%d page_tokens=%d is not a shape "
                "this kernel takes (groups of 1, 2, 4 or 8 heads; head_dim 64, 128 or 256; pages "
                "in multiples of 16)", n_heads, n_kv, head_dim, page_tokens);
    SIB_REQUIRE(rows > 0 && splits >= 1 && splits <= MAX_SPLITS,
                "attention_decode: rows=%d splits=%d (1 to %d)", rows, splits, MAX_SPLITS);
    SIB_REQUIRE(warps == 1 || warps == 2 || warps == 4 || warps == 8,
                "attention_decode: %d warps a block; 1, 2, 4 or 8", warps);
    SIB_REQUIRE(splits == 1 || (partial != nullptr && tickets != nullptr &&
                                ((uintptr_t)partial % 16) == 0),
                "attention_decode: %d splits need memory for their partial results and the "
                "ticket counters of the (row, kv head) pairs", splits);
    SIB_REQUIRE(k_pool && v_pool && page_table && max_pages > 0,
                "attention_decode: incomplete cache description");
    SIB_REQUIRE(ring_tokens >= 0 && ring_tokens % 16 == 0 && window >= 0,
                "attention_decode: ring=%d window=%d", ring_tokens, window);
    SIB_REQUIRE(q_stride % 8 == 0 && ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 &&
                    ((uintptr_t)v_pool % 16) == 0 && ((uintptr_t)out % 16) == 0,
                "attention_decode: operands must be 16-byte aligned");
    AttnDecodeArgs p{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool,
                     (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, partial, tickets, row_pos, row_seq,
                     seq_slot, page_table, q_stride, rows, n_heads, n_kv, max_pages, page_tokens,
                     ring_tokens, window, splits, scale, softcap, fresh};
    const long long blocks = (long long)rows * n_kv * splits;
    SIB_REQUIRE(blocks < (1ll << 31), "attention_decode: too many rows (%d)", rows);
    cudaStream_t s = (cudaStream_t)stream;
    const int G = n_heads / n_kv;
    const bool early_keys = fresh > 0 && rows == 1;
#define GO(HD, GG)                                                                                 \
    do {                                                                                           \
        if (warps == 8 && (size_t)warps * GG * (HD + 2) * sizeof(float) > 32 * 1024) {             \
            /* (with the kernel's own arrays these do not fit the default 48 KB) */                \
            cudaFuncSetAttribute(attention_decode_kernel<HD, GG, true, true>,                      \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,                      \
                                 (int)((size_t)warps * GG * (HD + 2) * sizeof(float)));            \
            cudaFuncSetAttribute(attention_decode_kernel<HD, GG, false, true>,                     \
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,                      \
                                 (int)((size_t)warps * GG * (HD + 2) * sizeof(float)));            \
        }                                                                                          \
        if (warps == 8 && early_keys)                                                              \
            sib_launch_chained(attention_decode_kernel<HD, GG, true, true>, dim3((unsigned)blocks), \
                               dim3(32 * warps), (size_t)warps * GG * (HD + 2) * sizeof(float), s, p); \
        else if (warps == 8)                                                                       \
            sib_launch_chained(attention_decode_kernel<HD, GG, false, true>, dim3((unsigned)blocks), \
                               dim3(32 * warps), (size_t)warps * GG * (HD + 2) * sizeof(float), s, p); \
        else if (early_keys)                                                                       \
            sib_launch_chained(attention_decode_kernel<HD, GG, true>, dim3((unsigned)blocks),      \
                               dim3(32 * warps), (size_t)warps * GG * (HD + 2) * sizeof(float), s, p); \
        else                                                                                       \
            sib_launch_chained(attention_decode_kernel<HD, GG, false>, dim3((unsigned)blocks),     \
                               dim3(32 * warps), (size_t)warps * GG * (HD + 2) * sizeof(float), s, p); \
    } while (0)
#define BY_G(HD)                  \
    do {                          \
        if (G == 1) GO(HD, 1);    \
        else if (G == 2) GO(HD, 2); \
        else if (G == 4) GO(HD, 4); \
        else GO(HD, 8);           \
    } while (0)
    if (head_dim == 64) BY_G(64);
    else if (head_dim == 128) BY_G(128);
    else BY_G(256);
#undef BY_G
#undef GO
    return sib_check_launch("attention_decode");
}

SIB_EXPORT int sib_attention_decode(
    const void* q, int q_stride, const void* k_pool, const void* v_pool, const int* page_table,
    int max_pages, int page_tokens, int ring_tokens, const int* row_pos, const int* row_seq,
    const int* seq_slot, void* out, float* partial, int* tickets, int rows, int n_heads, int n_kv,
    int head_dim, float scale, float softcap, int window, int splits, int warps, void* stream) {
    return attention_decode(q, q_stride, k_pool, v_pool, page_table, max_pages, page_tokens,
                            ring_tokens, row_pos, row_seq, seq_slot, out, partial, tickets, rows,
                            n_heads, n_kv, head_dim, scale, softcap, window, splits, warps, 0, stream);
}

// The same for a caller that knows how many positions per sequence the kernel before this
// one has written at most (`fresh`: the largest number of rows a sequence has in this step;
// the keys and values below them are older than that kernel and are fetched while it runs).
SIB_EXPORT int sib_attention_decode_fresh(
    const void* q, int q_stride, const void* k_pool, const void* v_pool, const int* page_table,
    int max_pages, int page_tokens, int ring_tokens, const int* row_pos, const int* row_seq,
    const int* seq_slot, void* out, float* partial, int* tickets, int rows, int n_heads, int n_kv,
    int head_dim, float scale, float softcap, int window, int splits, int warps, int fresh,
    void* stream) {
    SIB_REQUIRE(fresh >= 0, "attention_decode: %d fresh positions", fresh);
    return attention_decode(q, q_stride, k_pool, v_pool, page_table, max_pages, page_tokens,
                            ring_tokens, row_pos, row_seq, seq_slot, out, partial, tickets, rows,
                            n_heads, n_kv, head_dim, scale, softcap, window, splits, warps, fresh,
                            stream);
}

// ---------------------------------------------------------------------------
// The same kernels for callers that cannot allocate (attention_decode_no_alloc.h):
// the splits' partial results go to an array that is part of this library.
// ---------------------------------------------------------------------------
#include <mutex>

#include "attention_decode_no_alloc.h"

static __device__ __align__(256) float g_no_alloc_scratch[NO_ALLOC_SCRATCH_FLOATS];

// In host code the name g_no_alloc_scratch is only a handle; the address a kernel
// can use is looked up once per device and kept here.
static const int kMaxDevices = 64;
static float* g_no_alloc_address[kMaxDevices] = {};
static std::mutex g_no_alloc_mutex;

static int no_alloc_scratch_address(float** address) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= kMaxDevices) {
        sib_set_error("attention_decode_no_alloc: cannot tell the current device (%s)",
                      e != cudaSuccess ? cudaGetErrorString(e) : "index out of range");
        return e != cudaSuccess ? (int)e : -1;
    }
    std::lock_guard<std::mutex> guard(g_no_alloc_mutex);
    if (g_no_alloc_address[device] == nullptr) {
        void* found = nullptr;
        e = cudaGetSymbolAddress(&found, g_no_alloc_scratch);
        if (e != cudaSuccess || found == nullptr) {
            sib_set_error("attention_decode_no_alloc: cudaGetSymbolAddress failed on device %d: %s",
                          device, cudaGetErrorString(e));
            return e != cudaSuccess ? (int)e : -1;
        }
        g_no_alloc_address[device] = (float*)found;
    }
    *address = g_no_alloc_address[device];
    return 0;
}

// The ticket counters have a region of their own at the front of the array, of a fixed
// size, so that no call's partial results can land where another call's counters live.
static_assert(NO_ALLOC_TICKET_SLOTS % 64 == 0 && NO_ALLOC_TICKET_SLOTS < NO_ALLOC_SCRATCH_FLOATS,
              "the ticket region is a whole number of 256-byte lines inside the array");

SIB_EXPORT long long sib_attention_decode_no_alloc_floats(int rows, int n_heads, int head_dim,
                                                          int splits) {
    if (splits <= 1) return 0;
    return (long long)NO_ALLOC_TICKET_SLOTS + (long long)rows * n_heads * splits * (head_dim + 2);
}

SIB_EXPORT int sib_attention_decode_no_alloc(
    const void* q, int q_stride, const void* k_pool, const void* v_pool, const int* page_table,
    int max_pages, int page_tokens, int ring_tokens, const int* row_pos, const int* row_seq,
    const int* seq_slot, void* out, int rows, int n_heads, int n_kv, int head_dim, float scale,
    float softcap, int window, int splits, void* stream) {
    SIB_REQUIRE(rows >= 0 && n_heads > 0 && n_kv > 0 && head_dim > 0 && splits >= 1,
                "attention_decode_no_alloc: rows=%d heads=%d kv_heads=%d head_dim=%d splits=%d",
                rows, n_heads, n_kv, head_dim, splits);
    const long long need = sib_attention_decode_no_alloc_floats(rows, n_heads, head_dim, splits);
    SIB_REQUIRE(need <= (long long)NO_ALLOC_SCRATCH_FLOATS,
                "attention_decode_no_alloc: %d rows x %d heads x %d splits x (%d + 2) floats of "
                "partial results and the ticket counters come to %lld floats, the built-in array "
                "holds %u; use fewer splits or rows, or sib_attention_decode with memory of your own",
                rows, n_heads, splits, head_dim, need, NO_ALLOC_SCRATCH_FLOATS);
    SIB_REQUIRE(splits <= 1 || (long long)rows * n_kv <= (long long)NO_ALLOC_TICKET_SLOTS,
                "attention_decode_no_alloc: %d rows x %d kv heads need %lld ticket counters, the "
                "built-in array holds %u; use fewer rows, or sib_attention_decode with memory of "
                "your own", rows, n_kv, (long long)rows * n_kv, NO_ALLOC_TICKET_SLOTS);
    float* scratch = nullptr;
    const int rc = no_alloc_scratch_address(&scratch);   // the first call on a device sets it up
    if (rc) return rc;
    if (splits > 1) {
        // The counters this launch uses start at zero whatever an earlier launch left there
        // (one that failed midway does not put its counters back).  A memset on the call's
        // stream allocates nothing.
        cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)rows * n_kv * sizeof(int),
                                        (cudaStream_t)stream);
        if (e != cudaSuccess) {
            sib_set_error("attention_decode_no_alloc: clearing the ticket counters failed: %s",
                          cudaGetErrorString(e));
            return (int)e;
        }
    }
    return sib_attention_decode(q, q_stride, k_pool, v_pool, page_table, max_pages, page_tokens,
                                ring_tokens, row_pos, row_seq, seq_slot, out,
                                scratch + NO_ALLOC_TICKET_SLOTS, (int*)scratch, rows,
                                n_heads, n_kv, head_dim, scale, softcap, window, splits, 4, stream);
}
