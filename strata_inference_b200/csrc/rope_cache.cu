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
        bool keep = true;
        int cell = pos;
        if (p.ring_tokens > 0) {
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
    int threads = 32;
    while (threads < 128 && threads < head_dim / 2) threads *= 2;
    dim3 grid(rows, n_heads + 2 * n_kv);
    SIB_DISPATCH_DTYPE(dtype, (rope_store_kernel<T><<<grid, threads, 0, (cudaStream_t)stream>>>(p)));
    return sib_check_launch("rope_store");
}
