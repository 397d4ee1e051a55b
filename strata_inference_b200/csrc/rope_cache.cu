// Rotary position encoding of q and k, and the write of k and v into the
// paged cache, in one pass over the step's packed q|k|v rows.
//
// Rotation (angles in f32): pair (x[i], x[i + rot/2]) ("half-split") or
// (x[2i], x[2i+1]) ("interleaved"), angle = pos * inv_freq[i]:
//     x0' = x0 cos - x1 sin,   x1' = x0 sin + x1 cos
// Plain counterpart: tests/plain_gemma2.py rope_neox().
// Reference: src/backend/cpu.rs:1276-1322 (half-split), src/model/layer.rs:906-914
// (q and k only, position = cache length + row), src/model/cache.rs:210-244 (append).
//
// Cache layout of one layer: pool[page][kv_head][token_in_page][head_dim]; a
// sequence's page table maps (position / page_tokens) to a page, or for a ring
// ((position % ring_tokens) / page_tokens).  A ring keeps the last ring_tokens
// positions only, so rows older than that at the end of the step are not written
// (another row of the same step owns their cell).
#include "common.cuh"

struct RopeStoreArgs {
    void* qkv;                 // [rows, (n_heads + 2 n_kv) * head_dim], rotated in place
    const int* row_pos;        // [rows] absolute position
    const int* row_seq;        // [rows] index into the step's sequences
    const int* seq_slot;       // [seqs]
    const int* seq_end;        // [seqs] length after this step
    const float* inv_freq;     // [rot/2] or null
    void* k_pool;              // null: nothing is stored
    void* v_pool;
    const int* page_table;     // [slots, max_pages]
    int n_heads, n_kv, head_dim, rot, style;
    int max_pages, page_tokens, ring_tokens;
};

template <typename T>
__global__ void rope_store_kernel(RopeStoreArgs p) {
    pdl_trigger();
    pdl_wait();
    const int r = blockIdx.x, y = blockIdx.y;
    const int hd = p.head_dim;
    const int width = (p.n_heads + 2 * p.n_kv) * hd;
    T* x = (T*)p.qkv + (size_t)r * width + (size_t)y * hd;
    const int pos = p.row_pos[r];
    const bool is_v = y >= p.n_heads + p.n_kv;
    const bool is_kv = y >= p.n_heads;

    T* dst = nullptr;
    if (is_kv && p.k_pool) {
        const int b = p.row_seq[r];
        bool keep = p.seq_slot[b] >= 0;      // (a padding row's sequence holds no slot)
        int cell = pos;
        if (keep && p.ring_tokens > 0) {
            keep = pos >= p.seq_end[b] - p.ring_tokens;
            cell = pos % p.ring_tokens;
        }
        if (keep) {
            const int page = p.page_table[(size_t)p.seq_slot[b] * p.max_pages + cell / p.page_tokens];
            const int kvh = is_v ? y - p.n_heads - p.n_kv : y - p.n_heads;
            T* pool = (T*)(is_v ? p.v_pool : p.k_pool);
            dst = pool + (((size_t)page * p.n_kv + kvh) * p.page_tokens + cell % p.page_tokens) * hd;
        }
    }

    const int half = p.rot / 2;
    if (!is_v && half > 0) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const int i0 = p.style == 0 ? i : 2 * i;
            const int i1 = p.style == 0 ? i + half : 2 * i + 1;
            const float ang = (float)pos * p.inv_freq[i];
            const float c = cosf(ang), s = sinf(ang);
            const float x0 = to_f32(x[i0]), x1 = to_f32(x[i1]);
            const T y0 = from_f32<T>(x0 * c - x1 * s), y1 = from_f32<T>(x0 * s + x1 * c);
            x[i0] = y0;
            x[i1] = y1;
            if (dst) { dst[i0] = y0; dst[i1] = y1; }
        }
        if (dst)
            for (int i = p.rot + threadIdx.x; i < hd; i += blockDim.x) dst[i] = x[i];
    } else if (dst) {
        for (int i = threadIdx.x; i < hd; i += blockDim.x) dst[i] = x[i];
    }
}

// The common case in 16-byte accesses: bfloat16, half-split pairs, the whole
// head rotated.  One block per row; a thread takes 8 pairs (x[i..i+8) with
// x[i+half..i+half+8)) of a q or k head, or 8 elements of a v head.
// A row's units of work are dealt out over the threads of gridDim.y blocks.
// TABLE: the block first puts the row's cosines and sines (one pair per rotated pair of
// a head: the same for every head) into shared memory; else every unit takes its own.
template <bool TABLE>
__global__ void __launch_bounds__(128) rope_store_bf16_kernel(RopeStoreArgs p) {
    extern __shared__ float2 cs_table[];       // [head_dim / 2] (cos, sin), with TABLE
    pdl_trigger();
    const int r = blockIdx.x;
    const int first = blockIdx.y * blockDim.x + threadIdx.x, step = gridDim.y * blockDim.x;
    const int hd = p.head_dim, half = hd / 2;
    const int width = (p.n_heads + 2 * p.n_kv) * hd;
    __nv_bfloat16* row = (__nv_bfloat16*)p.qkv + (size_t)r * width;
    const int pos = p.row_pos[r];
    size_t cell_off = 0;
    bool keep = false;
    if (p.k_pool) {
        const int b = p.row_seq[r];
        int cell = pos;
        keep = p.seq_slot[b] >= 0;           // (a padding row's sequence holds no slot)
        if (keep && p.ring_tokens > 0) {
            keep = pos >= p.seq_end[b] - p.ring_tokens;
            cell = pos % p.ring_tokens;
        }
        if (keep) {
            const int page = p.page_table[(size_t)p.seq_slot[b] * p.max_pages + cell / p.page_tokens];
            cell_off = ((size_t)page * p.n_kv * p.page_tokens + cell % p.page_tokens) * hd;
        }
    }
    if (TABLE) {
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            const float ang = (float)pos * p.inv_freq[i];
            cs_table[i] = make_float2(cosf(ang), sinf(ang));
        }
        __syncthreads();
    }
    // (positions, slots and page tables are written by the host before the step: only from
    // here on does the kernel need what the kernel before it wrote)
    pdl_wait();
    const size_t head_step = (size_t)p.page_tokens * hd;    // between kv heads of a page
    const int per_head = half / 8;
    for (int u = first; u < (p.n_heads + p.n_kv) * per_head; u += step) {
        const int y = u / per_head, i0 = (u % per_head) * 8;
        __nv_bfloat16* x = row + (size_t)y * hd;
        const uint4 lo = *reinterpret_cast<const uint4*>(x + i0);
        const uint4 hi = *reinterpret_cast<const uint4*>(x + i0 + half);
        const uint32_t lw[4] = {lo.x, lo.y, lo.z, lo.w}, hw[4] = {hi.x, hi.y, hi.z, hi.w};
        uint32_t ol[4], oh[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float a[2] = {__uint_as_float(lw[k] << 16), __uint_as_float(lw[k] & 0xffff0000u)};
            float bq[2] = {__uint_as_float(hw[k] << 16), __uint_as_float(hw[k] & 0xffff0000u)};
            float ra[2], rb[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float c, s;
                if (TABLE) {
                    const float2 t = cs_table[i0 + 2 * k + e];
                    c = t.x;
                    s = t.y;
                } else {
                    const float ang = (float)pos * p.inv_freq[i0 + 2 * k + e];
                    c = cosf(ang);
                    s = sinf(ang);
                }
                ra[e] = a[e] * c - bq[e] * s;
                rb[e] = a[e] * s + bq[e] * c;
            }
            const __nv_bfloat162 pa = __floats2bfloat162_rn(ra[0], ra[1]);
            const __nv_bfloat162 pb = __floats2bfloat162_rn(rb[0], rb[1]);
            ol[k] = *reinterpret_cast<const uint32_t*>(&pa);
            oh[k] = *reinterpret_cast<const uint32_t*>(&pb);
        }
        const uint4 vlo = make_uint4(ol[0], ol[1], ol[2], ol[3]);
        const uint4 vhi = make_uint4(oh[0], oh[1], oh[2], oh[3]);
        *reinterpret_cast<uint4*>(x + i0) = vlo;
        *reinterpret_cast<uint4*>(x + i0 + half) = vhi;
        if (keep && y >= p.n_heads) {
            __nv_bfloat16* dst = (__nv_bfloat16*)p.k_pool + cell_off + (size_t)(y - p.n_heads) * head_step;
            *reinterpret_cast<uint4*>(dst + i0) = vlo;
            *reinterpret_cast<uint4*>(dst + i0 + half) = vhi;
        }
    }
    if (keep) {
        const int per_v = hd / 8;
        const __nv_bfloat16* v = row + (size_t)(p.n_heads + p.n_kv) * hd;
        for (int u = first; u < p.n_kv * per_v; u += step) {
            const int y = u / per_v, i0 = (u % per_v) * 8;
            __nv_bfloat16* dst = (__nv_bfloat16*)p.v_pool + cell_off + (size_t)y * head_step;
            *reinterpret_cast<uint4*>(dst + i0) = *reinterpret_cast<const uint4*>(v + (size_t)y * hd + i0);
        }
    }
}

SIB_EXPORT int sib_rope_store(void* qkv, int dtype, const int* row_pos, const int* row_seq,
                              const int* seq_slot, const int* seq_end, const float* inv_freq,
                              int rot, int style, void* k_pool, void* v_pool,
                              const int* page_table, int max_pages, int page_tokens,
                              int ring_tokens, int rows, int n_heads, int n_kv, int head_dim,
                              void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_heads >= 0 && n_kv >= 0 && n_heads + n_kv > 0 && head_dim > 0,
                "rope_store: rows=%d heads=%d kv=%d head_dim=%d", rows, n_heads, n_kv, head_dim);
    SIB_REQUIRE(rot >= 0 && rot <= head_dim && rot % 2 == 0,
                "rope_store: rotary size %d must be even and at most head_dim %d", rot, head_dim);
    SIB_REQUIRE(rot == 0 || inv_freq != nullptr, "rope_store: rotation without frequencies");
    SIB_REQUIRE(style == 0 || style == 1, "rope_store: unknown pairing %d", style);
    SIB_REQUIRE(k_pool == nullptr || (v_pool && page_table && page_tokens > 0 && max_pages > 0),
                "rope_store: incomplete cache description");
    SIB_REQUIRE(ring_tokens >= 0 && (ring_tokens == 0 || ring_tokens % page_tokens == 0),
                "rope_store: ring of %d tokens is not whole pages of %d", ring_tokens, page_tokens);
    RopeStoreArgs p{qkv, row_pos, row_seq, seq_slot, seq_end, inv_freq, k_pool, v_pool, page_table,
                    n_heads, n_kv, head_dim, rot, style, max_pages, page_tokens, ring_tokens};
    if (dtype == SIB_BF16 && style == 0 && rot == head_dim && head_dim % 16 == 0 &&
        ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 && ((uintptr_t)v_pool % 16) == 0) {
        // few rows (decoding): a row's heads spread over several small blocks, so that the
        // sines and cosines of a row are not one block's serial work
        const int units = (n_heads + n_kv) * (head_dim / 16);
        if (rows < 64)
            sib_launch_chained(rope_store_bf16_kernel<false>, dim3(rows, (units + 31) / 32), dim3(32),
                               0, (cudaStream_t)stream, p);
        else if (head_dim <= 4096)
            // many rows: a block per row shares one table of the row's cosines and sines
            sib_launch_chained(rope_store_bf16_kernel<true>, dim3(rows), dim3(128),
                               (size_t)(head_dim / 2) * sizeof(float2), (cudaStream_t)stream, p);
        else
            sib_launch_chained(rope_store_bf16_kernel<false>, dim3(rows), dim3(128), 0,
                               (cudaStream_t)stream, p);
        return sib_check_launch("rope_store");
    }
    int threads = 32;
    while (threads < 128 && threads < head_dim / 2) threads *= 2;
    dim3 grid(rows, n_heads + 2 * n_kv);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(rope_store_kernel<T>, grid, dim3(threads), 0,
                                                 (cudaStream_t)stream, p));
    return sib_check_launch("rope_store");
}

// ---------------------------------------------------------------------------
// The way back: keys and values of positions that a sequence already holds, copied from
// the pages into rows of a packed q|k|v buffer (row = position), so that a step that
// continues sequences with many tokens can run the prompt attention over "what was there
// + what came" (parts/attention.py).  Of sequence b the positions [from[b], upto[b]) go
// to rows row0[b] + position; the q columns of those rows are set to zero.
// ---------------------------------------------------------------------------
struct GatherArgs {
    __nv_bfloat16* packed;     // [rows, (n_heads + 2 n_kv) * head_dim]
    const __nv_bfloat16* k_pool;
    const __nv_bfloat16* v_pool;
    const int* page_table;     // [slots, max_pages]
    const int* seq_slot;       // [seqs]
    const int* seq_from;       // [seqs] first position to copy
    const int* seq_upto;       // [seqs] one past the last
    const int* seq_row0;       // [seqs] packed row of the sequence's position 0
    int n_heads, n_kv, head_dim;
    int max_pages, page_tokens, ring_tokens;
};

__global__ void __launch_bounds__(128) gather_kv_rows_kernel(GatherArgs p) {
    pdl_trigger();
    const int b = blockIdx.y;
    const int pos = p.seq_from[b] + blockIdx.x;
    pdl_wait();
    if (pos >= p.seq_upto[b]) return;
    const int hd = p.head_dim;
    const int width = (p.n_heads + 2 * p.n_kv) * hd;
    const int cell = p.ring_tokens > 0 ? pos % p.ring_tokens : pos;
    const int page = p.page_table[(size_t)p.seq_slot[b] * p.max_pages + cell / p.page_tokens];
    __nv_bfloat16* row = p.packed + (size_t)(p.seq_row0[b] + pos) * width;
    const int per_head = hd / 8;                 // 16-byte pieces of a head
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int u = threadIdx.x; u < p.n_heads * per_head; u += blockDim.x)
        reinterpret_cast<uint4*>(row)[u] = zero;
    for (int u = threadIdx.x; u < 2 * p.n_kv * per_head; u += blockDim.x) {
        const int which = u / (p.n_kv * per_head);          // 0: keys, 1: values
        const int kvh = (u / per_head) % p.n_kv, piece = u % per_head;
        const __nv_bfloat16* pool = which ? p.v_pool : p.k_pool;
        const __nv_bfloat16* src = pool + (((size_t)page * p.n_kv + kvh) * p.page_tokens +
                                           cell % p.page_tokens) * hd + 8 * piece;
        __nv_bfloat16* dst = row + (size_t)(p.n_heads + which * p.n_kv + kvh) * hd + 8 * piece;
        *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    }
}

// `most`: the most positions any sequence has to copy (the grid's width).
SIB_EXPORT int sib_gather_kv_rows(void* packed, const void* k_pool, const void* v_pool,
                                  const int* page_table, const int* seq_slot, const int* seq_from,
                                  const int* seq_upto, const int* seq_row0, int n_seqs, int most,
                                  int n_heads, int n_kv, int head_dim, int max_pages,
                                  int page_tokens, int ring_tokens, void* stream) {
    if (n_seqs == 0 || most <= 0) return 0;
    SIB_REQUIRE(n_seqs > 0 && n_seqs < 65536 && n_heads > 0 && n_kv > 0 && head_dim > 0 &&
                    head_dim % 8 == 0,
                "gather_kv_rows: seqs=%d heads=%d kv=%d head_dim=%d (a multiple of 8)", n_seqs, n_heads,
                n_kv, head_dim);
    SIB_REQUIRE(packed && k_pool && v_pool && page_table && seq_slot && seq_from && seq_upto && seq_row0 &&
                    page_tokens > 0 && max_pages > 0 && ring_tokens >= 0,
                "gather_kv_rows: incomplete description");
    SIB_REQUIRE(((uintptr_t)packed % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 &&
                    ((uintptr_t)v_pool % 16) == 0,
                "gather_kv_rows: buffers must be 16-byte aligned");
    GatherArgs p{(__nv_bfloat16*)packed, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool,
                 page_table, seq_slot, seq_from, seq_upto, seq_row0, n_heads, n_kv, head_dim,
                 max_pages, page_tokens, ring_tokens};
    sib_launch_chained(gather_kv_rows_kernel, dim3(most, n_seqs), dim3(128), 0, (cudaStream_t)stream, p);
    return sib_check_launch("gather_kv_rows");
}
