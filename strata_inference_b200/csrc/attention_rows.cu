// Attention of independent query rows over the paged cache and the step's
// own keys: the general kernel (any head size in steps of 16 up to 512, any
// grouping, 32-bit or bfloat16 storage, 32-bit arithmetic throughout).
//
// For the query row at absolute position p of sequence b and query head h
// (key/value head g = h / (n_heads / n_kv)):
//     s_j = scale * <q_h, k_{g,j}>;  if cap > 0: s_j = cap * tanh(s_j / cap)
//     visible j: max(0, p - window + 1) <= j <= p   (window 0: all j <= p)
//     o = sum_j softmax(s)_j v_{g,j}
// Keys at positions >= seq_start[b] (this step's own rows) are read from the
// step's packed k/v rows when those are given; earlier ones from the cache.
// With splits > 1 each (row, head) is cut into `splits` runs of keys whose
// partial (max, sum, accumulator) go to scratch memory and are merged, in
// split order, by attention_combine.
//
// Plain counterpart: tests/plain_gemma2.py attention().
// Reference: src/backend/cpu.rs:1352-1434 (decode), src/model/layer.rs:1030-1066
// (order scale, cap, mask), src/backend/cuda/kernels.rs:3243-3262 (window bounds).
#include "common.cuh"

struct AttnRowsArgs {
    const void* q;          // row r, head h at q + r * q_stride + h * head_dim
    const void* k_new;      // this step's keys (null: everything comes from the cache)
    const void* v_new;
    const void* k_pool;     // may be null when every key is in k_new
    const void* v_pool;
    void* out;              // [rows, n_heads * head_dim]
    float* partial;         // [rows, n_heads, splits, head_dim + 2] when splits > 1
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_start;   // position of the sequence's first row in this step
    const int* seq_row0;    // packed row index of that first row
    const int* page_table;
    int q_stride, kv_stride;
    int rows, n_heads, n_kv, head_dim;
    int max_pages, page_tokens, ring_tokens;
    int window, splits;
    float scale, softcap;
};

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&o)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&o)[8]) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            o[2 * i] = __uint_as_float(w[i] << 16);
            o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

template <typename T>
__device__ __forceinline__ const T* key_ptr(const AttnRowsArgs& p, const T* fresh, const T* pool,
                                            int j, int start, int row0, int slot, int g) {
    if (fresh && j >= start)
        return fresh + (size_t)(row0 + (j - start)) * p.kv_stride + (size_t)g * p.head_dim;
    const int cell = p.ring_tokens > 0 ? j % p.ring_tokens : j;
    const int page = p.page_table[(size_t)slot * p.max_pages + cell / p.page_tokens];
    return pool + (((size_t)page * p.n_kv + g) * p.page_tokens + cell % p.page_tokens) * p.head_dim;
}

// One warp per (row, head, split).  Lane l owns the 16-byte vectors number
// l, l + 32, ... of the head (NI of them at most).
template <typename T, int NI>
__global__ void __launch_bounds__(128) attention_rows_kernel(AttnRowsArgs p) {
    constexpr int V = Vec16<T>::N;
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long unit = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (unit >= (long long)p.rows * p.n_heads * p.splits) return;
    const int split = (int)(unit % p.splits);
    const int h = (int)((unit / p.splits) % p.n_heads);
    const int r = (int)(unit / ((long long)p.splits * p.n_heads));
    const int g = h / (p.n_heads / p.n_kv);
    const int hd = p.head_dim;

    const int pos = p.row_pos[r];
    const int b = p.row_seq[r];
    const int slot = p.seq_slot[b];
    const int start = p.seq_start[b];
    const int row0 = p.seq_row0[b];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int n = pos - lo + 1;
    const int chunk = (n + p.splits - 1) / p.splits;
    const int j0 = lo + split * chunk;
    const int j1 = min(j0 + chunk, pos + 1);

    bool live[NI];
    float qv[NI][V], acc[NI][V];
    const T* qp = (const T*)p.q + (size_t)r * p.q_stride + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < NI; ++i) {
        const int d = (lane + 32 * i) * V;
        live[i] = d < hd;
#pragma unroll
        for (int e = 0; e < V; ++e) { qv[i][e] = 0.f; acc[i][e] = 0.f; }
        if (live[i]) Vec16<T>::load(qp + d, qv[i]);
    }

    float m = -INFINITY, l = 0.f;
    const T* kf = (const T*)p.k_new;
    const T* vf = (const T*)p.v_new;
    const T* kpool = (const T*)p.k_pool;
    const T* vpool = (const T*)p.v_pool;

    constexpr int U = 4;  // keys in flight per iteration
    for (int j = j0; j < j1; j += U) {
        float s[U];
        float kv[U][NI][V];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (j + u < j1) {
                const T* kp = key_ptr<T>(p, kf, kpool, j + u, start, row0, slot, g);
#pragma unroll
                for (int i = 0; i < NI; ++i)
                    if (live[i]) Vec16<T>::load(kp + (lane + 32 * i) * V, kv[u][i]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            float d = 0.f;
            if (j + u < j1) {
#pragma unroll
                for (int i = 0; i < NI; ++i)
                    if (live[i]) {
#pragma unroll
                        for (int e = 0; e < V; ++e) d += qv[i][e] * kv[u][i][e];
                    }
            }
            s[u] = d;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < U; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
        }
        float mx = m;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (j + u < j1) {
                float t = s[u] * p.scale;
                if (p.softcap > 0.f) t = p.softcap * tanhf(t / p.softcap);
                s[u] = t;
                mx = fmaxf(mx, t);
            } else {
                s[u] = -INFINITY;
            }
        }
        const float corr = expf(m - mx);  // m = -inf on the first pass: 0
        m = mx;
        l *= corr;
#pragma unroll
        for (int i = 0; i < NI; ++i)
#pragma unroll
            for (int e = 0; e < V; ++e) acc[i][e] *= corr;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (j + u < j1) {
                const T* vp = key_ptr<T>(p, vf, vpool, j + u, start, row0, slot, g);
#pragma unroll
                for (int i = 0; i < NI; ++i)
                    if (live[i]) Vec16<T>::load(vp + (lane + 32 * i) * V, kv[u][i]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (j + u < j1) {
                const float w = expf(s[u] - m);
                l += w;
#pragma unroll
                for (int i = 0; i < NI; ++i)
                    if (live[i]) {
#pragma unroll
                        for (int e = 0; e < V; ++e) acc[i][e] += w * kv[u][i][e];
                    }
            }
        }
    }

    if (p.splits == 1) {
        const float inv = 1.0f / l;
        T* op = (T*)p.out + (size_t)r * p.n_heads * hd + (size_t)h * hd;
#pragma unroll
        for (int i = 0; i < NI; ++i)
            if (live[i]) {
#pragma unroll
                for (int e = 0; e < V; ++e) op[(lane + 32 * i) * V + e] = from_f32<T>(acc[i][e] * inv);
            }
    } else {
        float* pp = p.partial + (((size_t)r * p.n_heads + h) * p.splits + split) * (hd + 2);
        if (lane == 0) { pp[0] = m; pp[1] = l; }
#pragma unroll
        for (int i = 0; i < NI; ++i)
            if (live[i]) {
#pragma unroll
                for (int e = 0; e < V; ++e) pp[2 + (lane + 32 * i) * V + e] = acc[i][e];
            }
    }
}

// out[r, h, :] = sum_s acc_s e^{m_s - M} / sum_s l_s e^{m_s - M}, s in split order.
template <typename T>
__global__ void attention_combine_kernel(const float* __restrict__ partial, T* __restrict__ out,
                                         int splits, int head_dim, int groups) {
    extern __shared__ float weight[];   // [splits] e^{m_s - M}, 0 for an empty split
    pdl_trigger();
    pdl_wait();
    const size_t unit = blockIdx.x;     // r * n_heads + h
    const float* pp = partial + unit * splits * (head_dim + 2);
    __shared__ float scratch[33];
    // thread s takes split s: the (max, sum) pairs are read in one round of loads
    float mine = -INFINITY;
    for (int s = threadIdx.x; s < splits; s += blockDim.x)
        mine = fmaxf(mine, pp[(size_t)s * (head_dim + 2)]);
    mine = warp_max(mine);
    if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = mine;
    __syncthreads();
    float M = -INFINITY;
    for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) M = fmaxf(M, scratch[w]);
    float part = 0.f;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float* ps = pp + (size_t)s * (head_dim + 2);
        const float w = ps[1] > 0.f ? expf(ps[0] - M) : 0.f;
        weight[s] = w;
        part += ps[1] * w;
    }
    const float L = block_sum(part, scratch);   // also makes weight[] visible to all
    const float inv = 1.0f / L;
    // `groups` groups of threads take alternating splits; a thread owns two dimensions.
    // An empty split wrote zeros and has weight 0: no branch, so the loads overlap.
    float2* sums = reinterpret_cast<float2*>(weight + ((splits + 1) & ~1));
    const int nv = head_dim / 2;
    const int grp = threadIdx.x / nv, v = threadIdx.x % nv;
    if (grp < groups) {
        float2 a = make_float2(0.f, 0.f);
#pragma unroll 8
        for (int s = grp; s < splits; s += groups) {
            const float2 x =
                *reinterpret_cast<const float2*>(pp + (size_t)s * (head_dim + 2) + 2 + 2 * v);
            a.x += x.x * weight[s];
            a.y += x.y * weight[s];
        }
        sums[grp * nv + v] = a;
    }
    __syncthreads();
    if (grp == 0) {
        float2 a = sums[v];
        for (int k = 1; k < groups; ++k) {     // in group order
            a.x += sums[k * nv + v].x;
            a.y += sums[k * nv + v].y;
        }
        out[unit * head_dim + 2 * v] = from_f32<T>(a.x * inv);
        out[unit * head_dim + 2 * v + 1] = from_f32<T>(a.y * inv);
    }
}

struct CombineShape {
    int threads, groups;
    size_t smem;
};
static CombineShape combine_shape(int splits, int head_dim) {
    const int nv = head_dim / 2;
    int groups = 512 / nv;
    groups = groups < 1 ? 1 : (groups > 8 ? 8 : groups);
    CombineShape c;
    c.groups = groups;
    c.threads = (groups * nv + 31) / 32 * 32;
    c.smem = (size_t)((splits + 1) & ~1) * sizeof(float) + (size_t)groups * nv * sizeof(float2);
    return c;
}

// Shared with attention_decode.cu, whose partial results have the same layout.
int sib_launch_attention_combine_bf16(const float* partial, void* out, int units, int splits,
                                      int head_dim, cudaStream_t s) {
    const CombineShape c = combine_shape(splits, head_dim);
    sib_launch_chained(attention_combine_kernel<__nv_bfloat16>, dim3(units), dim3(c.threads), c.smem,
                       s, partial, (__nv_bfloat16*)out, splits, head_dim, c.groups);
    return sib_check_launch("attention_combine");
}

SIB_EXPORT long long sib_attention_rows_scratch_bytes(int rows, int n_heads, int head_dim,
                                                      int splits) {
    if (splits <= 1) return 0;
    return (long long)rows * n_heads * splits * (head_dim + 2) * (long long)sizeof(float);
}

SIB_EXPORT int sib_attention_rows(
    const void* q, int q_stride, const void* k_new, const void* v_new, int kv_stride,
    const void* k_pool, const void* v_pool, const int* page_table, int max_pages, int page_tokens,
    int ring_tokens, const int* row_pos, const int* row_seq, const int* seq_slot,
    const int* seq_start, const int* seq_row0, void* out, float* partial, int dtype, int rows,
    int n_heads, int n_kv, int head_dim, float scale, float softcap, int window, int splits,
    void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && n_heads > 0 && n_kv > 0 && n_heads % n_kv == 0,
                "attention_rows: rows=%d heads=%d kv_heads=%d", rows, n_heads, n_kv);
    SIB_REQUIRE(head_dim >= 16 && head_dim % 16 == 0 && head_dim <= 512,
                "attention_rows: head_dim=%d must be a multiple of 16 between 16 and 512", head_dim);
    SIB_REQUIRE(splits >= 1 && (splits == 1 || partial != nullptr),
                "attention_rows: splits=%d without scratch memory", splits);
    SIB_REQUIRE((k_new != nullptr) == (v_new != nullptr) && (k_pool != nullptr) == (v_pool != nullptr),
                "attention_rows: keys and values must come from the same places");
    SIB_REQUIRE(k_new != nullptr || k_pool != nullptr, "attention_rows: no keys given");
    SIB_REQUIRE(k_pool == nullptr || (page_table && page_tokens > 0 && max_pages > 0),
                "attention_rows: incomplete cache description");
    SIB_REQUIRE(window >= 0 && ring_tokens >= 0, "attention_rows: window=%d ring=%d", window,
                ring_tokens);
    const int esz = dtype == SIB_F32 ? 4 : 2;
    SIB_REQUIRE(((size_t)q_stride * esz) % 16 == 0 && ((size_t)kv_stride * esz) % 16 == 0 &&
                    ((uintptr_t)q % 16) == 0 && ((uintptr_t)k_new % 16) == 0 &&
                    ((uintptr_t)v_new % 16) == 0 && ((uintptr_t)k_pool % 16) == 0 &&
                    ((uintptr_t)v_pool % 16) == 0,
                "attention_rows: rows must start on 16-byte boundaries");
    AttnRowsArgs p{q, k_new, v_new, k_pool, v_pool, out, partial, row_pos, row_seq, seq_slot,
                   seq_start, seq_row0, page_table, q_stride, kv_stride, rows, n_heads, n_kv,
                   head_dim, max_pages, page_tokens, ring_tokens, window, splits, scale, softcap};
    const long long units = (long long)rows * n_heads * splits;
    const long long blocks = (units + 3) / 4;
    SIB_REQUIRE(blocks < (1ll << 31), "attention_rows: too many rows (%d)", rows);
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = 16 / esz;
    const int ni = (head_dim + 32 * vec - 1) / (32 * vec);
#define LAUNCH(NI) \
    sib_launch_chained(attention_rows_kernel<T, NI>, dim3((unsigned)blocks), dim3(128), 0, s, p)
    SIB_DISPATCH_DTYPE(dtype, {
        if (ni == 1) LAUNCH(1);
        else if (ni == 2) LAUNCH(2);
        else LAUNCH(4);
    });
#undef LAUNCH
    int rc = sib_check_launch("attention_rows");
    if (rc || splits == 1) return rc;
    const CombineShape c = combine_shape(splits, head_dim);
    SIB_DISPATCH_DTYPE(dtype, sib_launch_chained(attention_combine_kernel<T>, dim3(rows * n_heads),
                                                 dim3(c.threads), c.smem, s, partial, (T*)out,
                                                 splits, head_dim, c.groups));
    return sib_check_launch("attention_combine");
}
