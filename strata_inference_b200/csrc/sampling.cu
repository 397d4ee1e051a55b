// Next-token selection on the device: greedy, or temperature / top-k / top-p
// sampling with one xorshift64 generator per sequence.
//
// Order of the operations (src/engine/sampler.rs:82-152): z = logit / T; if
// top-k is on, keep the k largest z (ties: lowest index first); softmax over
// what is kept; if top-p is on, keep the shortest prefix, by descending
// probability, whose mass reaches p, and renormalise; draw r in [0, 1) and take
// the first kept token whose running sum exceeds r.  The running sum goes by
// token index when no filter is on and by descending z (ties by index) when one
// is, as in the reference, whose filters sort their candidates.  Greedy takes
// the first maximum (src/engine/sampler.rs:61-71).  The generator is
// src/engine/sampler.rs:36-58: x ^= x << 13; x ^= x >> 7; x ^= x << 17;
// r = (x >> 40) / 2^24.
// Plain counterpart: tests/plain_gemma2.py sample_token(), argmax(), XorShift64.
//
// The filtered modes never sort: the k-th largest value, the value at which
// the mass reaches p and the value the draw lands on are each found by 32
// rounds of bisection on the order-preserving integer image of z, each round
// one pass over the row.
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ uint32_t order_key(float z) {
    const uint32_t u = __float_as_uint(z);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct ArgMax {
    float v;
    int i;
};
__device__ __forceinline__ ArgMax better(ArgMax a, ArgMax b) {
    // larger value wins; equal values: the lower index
    if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
    return a;
}

__device__ ArgMax block_argmax(ArgMax a, ArgMax* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ArgMax b;
        b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
        b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
        a = better(a, b);
    }
    __syncthreads();
    if (lane == 0) scratch[warp] = a;
    __syncthreads();
    if (warp == 0) {
        ArgMax t = lane < (int)(blockDim.x >> 5) ? scratch[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ArgMax b;
            b.v = __shfl_xor_sync(0xffffffffu, t.v, o);
            b.i = __shfl_xor_sync(0xffffffffu, t.i, o);
            t = better(t, b);
        }
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

struct Tally {       // elements at or above a threshold
    float mass;      // sum of exp(z - max)
    int count;
};

struct SampleArgs {
    const float* logits;   // [rows, stride]
    long long stride;
    int vocab;
    float temperature;
    int top_k;
    float top_p;
    unsigned long long* rng;  // generator states, advanced by one draw
    const int* rng_index;     // [rows] which state a row uses (null: its own number)
    int* out;                 // [rows]
};

// Block-wide sums of (mass, count); every thread gets the result.
__device__ Tally block_tally(Tally t, float* fs, int* is) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        t.mass += __shfl_xor_sync(0xffffffffu, t.mass, o);
        t.count += __shfl_xor_sync(0xffffffffu, t.count, o);
    }
    __syncthreads();
    if (lane == 0) { fs[warp] = t.mass; is[warp] = t.count; }
    __syncthreads();
    if (warp == 0) {
        float m = lane < (int)(blockDim.x >> 5) ? fs[lane] : 0.f;
        int c = lane < (int)(blockDim.x >> 5) ? is[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            m += __shfl_xor_sync(0xffffffffu, m, o);
            c += __shfl_xor_sync(0xffffffffu, c, o);
        }
        if (lane == 0) { fs[32] = m; is[32] = c; }
    }
    __syncthreads();
    Tally r;
    r.mass = fs[32];
    r.count = is[32];
    return r;
}

// Index of the `rank`-th (0-based) element, in index order, whose key equals `key`.
__device__ int nth_with_key(const float* row, int vocab, float inv_t, uint32_t key, int rank,
                            int* is, int* result) {
    const int per = (vocab + blockDim.x - 1) / blockDim.x;
    const int lo = min(vocab, (int)threadIdx.x * per), hi = min(vocab, lo + per);
    int mine = 0;
    for (int i = lo; i < hi; ++i) mine += order_key(row[i] * inv_t) == key;
    __syncthreads();
    is[threadIdx.x] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int w = 0; w < (int)blockDim.x; ++w) { const int c = is[w]; is[w] = run; run += c; }
        *result = -1;
    }
    __syncthreads();
    const int before = is[threadIdx.x];
    if (rank >= before && rank < before + mine) {
        int seen = before;
        for (int i = lo; i < hi; ++i)
            if (order_key(row[i] * inv_t) == key) {
                if (seen == rank) { *result = i; break; }
                ++seen;
            }
    }
    __syncthreads();
    return *result;
}

__global__ void __launch_bounds__(SAMPLE_THREADS) sample_rows_kernel(SampleArgs p) {
    __shared__ ArgMax am[33];
    __shared__ float fs[33];
    __shared__ int is[SAMPLE_THREADS];
    __shared__ int is2[33];
    __shared__ int result;
    __shared__ float draw;
    pdl_trigger();
    pdl_wait();
    const float* row = p.logits + (size_t)blockIdx.x * p.stride;
    const int V = p.vocab;

    ArgMax a{-INFINITY, 0x7fffffff};
    for (int i = threadIdx.x; i < V; i += blockDim.x) a = better(a, ArgMax{row[i], i});
    a = block_argmax(a, am);
    if (p.temperature <= 0.f) {
        if (threadIdx.x == 0) p.out[blockIdx.x] = a.i == 0x7fffffff ? 0 : a.i;
        return;
    }
    // The reference divides by T; 1/T times z differs from that in the last bit
    // at most, and every pass below uses the same product.
    const float inv_t = 1.0f / p.temperature;
    const float zmax = a.v * inv_t;

    if (threadIdx.x == 0) {
        const int which = p.rng_index ? p.rng_index[blockIdx.x] : (int)blockIdx.x;
        unsigned long long x = p.rng[which];
        x ^= x << 13;
        x ^= x >> 7;
        x ^= x << 17;
        p.rng[which] = x;
        draw = (float)(x >> 40) / 16777216.0f;
    }
    __syncthreads();
    const float r = draw;

    const bool use_k = p.top_k > 0 && p.top_k < V;
    const bool use_p = p.top_p < 1.0f;

    if (!use_k && !use_p) {
        // running sum by token index over contiguous runs, one run per thread
        const int per = (V + blockDim.x - 1) / blockDim.x;
        const int lo = min(V, (int)threadIdx.x * per), hi = min(V, lo + per);
        float mine = 0.f;
        for (int i = lo; i < hi; ++i) mine += expf(row[i] * inv_t - zmax);
        __shared__ float runs[SAMPLE_THREADS];
        runs[threadIdx.x] = mine;
        __syncthreads();
        if (threadIdx.x == 0) {
            float run = 0.f;
            for (int w = 0; w < (int)blockDim.x; ++w) { const float c = runs[w]; runs[w] = run; run += c; }
            fs[0] = run;
            result = V - 1;  // the reference's fallback: the last candidate
        }
        __syncthreads();
        const float target = r * fs[0];
        const float before = runs[threadIdx.x];
        if (hi > lo && target >= before && target < before + mine) {
            float cum = before;
            int pick = hi - 1;
            for (int i = lo; i < hi; ++i) {
                cum += expf(row[i] * inv_t - zmax);
                if (target < cum) { pick = i; break; }
            }
            result = pick;
        }
        __syncthreads();
        if (threadIdx.x == 0) p.out[blockIdx.x] = result;
        return;
    }

    // ---- filtered modes: thresholds on the ordered keys ------------------
    // kth: key of the k-th largest z; k_ties: how many elements equal to it are kept.
    uint32_t kth = 0;
    int k_ties = 0x7fffffff;
    if (use_k) {
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            Tally t{0.f, 0};
            for (int i = threadIdx.x; i < V; i += blockDim.x) t.count += order_key(row[i] * inv_t) >= cand;
            t = block_tally(t, fs, is2);
            if (t.count >= p.top_k) prefix = cand;
        }
        kth = prefix;
        Tally t{0.f, 0};
        for (int i = threadIdx.x; i < V; i += blockDim.x) t.count += order_key(row[i] * inv_t) > kth;
        t = block_tally(t, fs, is2);
        k_ties = p.top_k - t.count;
    }
    // mass of the kept set after top-k
    float q_kth = 0.f;   // exp(z - max) of one element equal to kth
    Tally all{0.f, 0};
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float z = row[i] * inv_t;
        const uint32_t key = order_key(z);
        if (key > kth || !use_k) all.mass += expf(z - zmax);
        if (use_k && key == kth) q_kth = expf(z - zmax);
    }
    {
        // every thread that saw an element equal to kth computed the same q_kth
        __syncthreads();
        if (threadIdx.x == 0) draw = 0.f;
        __syncthreads();
        if (q_kth > 0.f) draw = q_kth;
        __syncthreads();
        q_kth = draw;
    }
    all = block_tally(all, fs, is2);
    float Z = all.mass + (use_k ? (float)k_ties * q_kth : 0.f);

    // mass(c) = kept mass of keys >= c, in units of exp(z - max)
    // A key equal to kth contributes at most k_ties elements.
    auto mass_at_least = [&](uint32_t c, bool strict_only) {
        Tally t{0.f, 0};
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float z = row[i] * inv_t;
            const uint32_t key = order_key(z);
            const bool in = use_k ? key > kth : true;
            if (in && (strict_only ? key > c : key >= c)) { t.mass += expf(z - zmax); t.count += 1; }
        }
        t = block_tally(t, fs, is2);
        if (use_k && (strict_only ? kth > c : kth >= c)) { t.mass += (float)k_ties * q_kth; t.count += k_ties; }
        return t;
    };

    // top-p: the key at which the running mass (descending) first reaches p * Z
    uint32_t pth = 0;          // keys > pth are kept whole
    int p_ties = 0x7fffffff;   // elements equal to pth that are kept
    float Z2 = Z;
    if (use_p) {
        const float want = p.top_p * Z;
        uint32_t prefix = 0;
        for (int bit = 31; bit >= 0; --bit) {
            const uint32_t cand = prefix | (1u << bit);
            if (mass_at_least(cand, false).mass >= want) prefix = cand;
        }
        pth = prefix;
        const Tally above = mass_at_least(pth, true);
        const Tally upto = mass_at_least(pth, false);
        const int ties = upto.count - above.count;
        const float q = ties > 0 ? (upto.mass - above.mass) / (float)ties : 0.f;
        int need = ties;
        if (q > 0.f) {
            need = (int)ceilf((want - above.mass) / q);
            need = max(1, min(need, ties));
        }
        p_ties = need;
        Z2 = above.mass + (float)need * q;
        if (upto.mass < want) { pth = 0; p_ties = 0x7fffffff; Z2 = Z; }  // never reached: keep all
    }

    // the draw: first element, by descending key then index, whose running mass exceeds r * Z2
    const float target = r * Z2;
    uint32_t prefix = 0;
    for (int bit = 31; bit >= 0; --bit) {
        const uint32_t cand = prefix | (1u << bit);
        if (mass_at_least(cand, false).mass > target) prefix = cand;
    }
    // keys below the filters' thresholds are not candidates
    uint32_t floor_key = 0;
    if (use_k) floor_key = kth;
    if (use_p && pth > floor_key) floor_key = pth;
    uint32_t hit = prefix < floor_key ? floor_key : prefix;
    const Tally above = mass_at_least(hit, true);
    const Tally upto = mass_at_least(hit, false);
    int ties = upto.count - above.count;
    const float q = ties > 0 ? (upto.mass - above.mass) / (float)ties : 0.f;
    if (use_p && hit == pth) ties = min(ties, p_ties);
    int rank = q > 0.f ? (int)floorf((target - above.mass) / q) : 0;
    rank = max(0, min(rank, ties - 1));
    const int tok = nth_with_key(row, V, inv_t, hit, rank, is, &result);
    if (threadIdx.x == 0) p.out[blockIdx.x] = tok >= 0 ? tok : a.i;
}

SIB_EXPORT int sib_sample_rows(const float* logits, long long stride, int rows, int vocab,
                               float temperature, int top_k, float top_p,
                               unsigned long long* rng, const int* rng_index, int* out,
                               void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && vocab > 0 && stride >= vocab, "sample_rows: rows=%d vocab=%d", rows, vocab);
    SIB_REQUIRE(temperature <= 0.f || rng != nullptr, "sample_rows: sampling needs generator states");
    SIB_REQUIRE(top_k >= 0 && top_p > 0.f, "sample_rows: top_k=%d top_p=%f", top_k, top_p);
    SampleArgs p{logits, stride, vocab, temperature, top_k, top_p, rng, rng_index, out};
    sib_launch_chained(sample_rows_kernel, dim3(rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream, p);
    return sib_check_launch("sample_rows");
}
