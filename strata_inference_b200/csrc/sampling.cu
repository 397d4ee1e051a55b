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
// Layout of the work: a row of logits is shared by a cluster of 8 blocks, each
// owning a contiguous eighth of the vocabulary; partial results meet in the
// first block's shared memory (distributed shared memory) once per pass.
// The filtered modes never sort.  "The k-th largest z", "the z at which the
// running mass reaches p" and "the z the draw lands on" are each a search for
// where a running count or mass, taken in descending order, crosses a target;
// each is done by a radix walk over the order-preserving integer image of z,
// 4 bits a pass (16 buckets of count and mass per pass, 8 passes a search).
// All sums are taken in a fixed order, so a draw is reproducible.
// With top-k on and few candidates (at most SAMPLE_LIST at or above the k-th key, ties
// included) only the first of the three searches runs, without masses; the candidates are
// gathered into a list, sorted and walked one after the other (sample_from_short_list).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

#define SAMPLE_CLUSTER 8
#define SAMPLE_THREADS 512
#define SAMPLE_WARPS (SAMPLE_THREADS / 32)
#define SAMPLE_LIST 256     // a top-k set of at most this many candidates is sorted and walked as a list

__device__ __forceinline__ uint32_t order_key(float z) {
    const uint32_t u = __float_as_uint(z);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_value(uint32_t key) {      // the z of a key
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

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

// What the blocks of a cluster exchange in one pass: 16 buckets of (count, mass),
// or any 32 numbers.  Two buffers alternate so that one cluster barrier a pass is enough.
struct Exchange {
    float f[2][SAMPLE_CLUSTER][16];
    int i[2][SAMPLE_CLUSTER][16];
};

struct SampleShared {
    Exchange xchg;                       // used in the cluster's first block
    float bins_f[16][SAMPLE_THREADS];    // per-thread private buckets
    int bins_i[16][SAMPLE_THREADS];
    float tot_f[16];
    int tot_i[16];
    float warp_f[SAMPLE_WARPS];
    int warp_i[SAMPLE_WARPS];
    int scan[SAMPLE_THREADS];
    float scan_f[SAMPLE_THREADS];
    int result;
    float before_f, total_f;
    // the candidates of a short top-k list (used in the cluster's first block)
    float list_z[SAMPLE_LIST];
    int list_i[SAMPLE_LIST];
    float sorted_z[SAMPLE_LIST];
    int sorted_i[SAMPLE_LIST];
    int list_n;
};

struct Cluster {
    cg::cluster_group g;
    SampleShared* sh;       // this block's
    SampleShared* first;    // the first block's (remote unless rank == 0)
    int rank;
    int pass;
};

// Sum the 16 per-thread buckets over the block (fixed order), then over the cluster
// (block order).  Afterwards sh->tot_f / tot_i hold the cluster-wide totals in every
// block, and the exchange buffer of this pass ((pass - 1) & 1 after the call) still
// holds every block's own sums.
__device__ void cluster_bucket_totals(Cluster& c) {
    SampleShared* sh = c.sh;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    {   // warp w sums bucket w over all threads
        float f = 0.f;
        int n = 0;
        for (int t = lane; t < SAMPLE_THREADS; t += 32) {
            f += sh->bins_f[warp][t];
            n += sh->bins_i[warp][t];
        }
        f = warp_sum(f);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) n += __shfl_xor_sync(0xffffffffu, n, o);
        const int buf = c.pass & 1;
        if (lane == 0) {
            c.first->xchg.f[buf][c.rank][warp] = f;
            c.first->xchg.i[buf][c.rank][warp] = n;
        }
    }
    c.g.sync();
    if (threadIdx.x < 16) {
        const int buf = c.pass & 1;
        float f = 0.f;
        int n = 0;
        for (int b = 0; b < SAMPLE_CLUSTER; ++b) {
            f += c.first->xchg.f[buf][b][threadIdx.x];
            n += c.first->xchg.i[buf][b][threadIdx.x];
        }
        sh->tot_f[threadIdx.x] = f;
        sh->tot_i[threadIdx.x] = n;
    }
    __syncthreads();
    c.pass++;
}

// A set of candidates in descending order of key: every element with key > floor_key,
// followed by `floor_ties` elements equal to floor_key of mass `floor_q` each.
struct Kept {
    uint32_t floor_key;
    int floor_ties;
    float floor_q;
};

struct Crossing {
    uint32_t key;      // the key at which the running count / mass crosses the target
    int above_count;   // kept elements with a larger key
    float above_mass;
    int ties;          // kept elements with exactly this key
    float q;           // mass of one of them
    float total_mass;  // mass of the whole kept set (from the first pass)
    bool few;          // the walk stopped early: `key` is the lowest key of a bucket that, with
                       // everything above it, holds at most the asked-for number of elements
};

// Walk the radix tree of keys, 4 bits a level, towards the element where, in
// descending order, the running count reaches `want_count` (by_mass == false), or the
// running mass reaches (inclusive) / exceeds (!inclusive) fraction x (mass of the set).
__device__ Crossing find_crossing(Cluster& c, const float* row, int lo, int hi, float inv_t,
                                  float zmax, const Kept& kept, bool by_mass, int want_count,
                                  float fraction, bool inclusive, bool with_mass = true,
                                  int few_enough = 0) {
    SampleShared* sh = c.sh;
    Crossing r;
    r.key = 0;
    r.above_count = 0;
    r.above_mass = 0.f;
    r.ties = 0;
    r.q = 0.f;
    r.total_mass = 0.f;
    r.few = false;
    float want_mass = 0.f;
    for (int level = 0; level < 8; ++level) {
        const int shift = 28 - 4 * level;
        const uint32_t path_mask = level == 0 ? 0u : (0xffffffffu << (shift + 4));
#pragma unroll
        for (int b = 0; b < 16; ++b) {
            sh->bins_f[b][threadIdx.x] = 0.f;
            sh->bins_i[b][threadIdx.x] = 0;
        }
        for (int i = lo + threadIdx.x; i < hi; i += SAMPLE_THREADS) {
            const float z = row[i] * inv_t;
            const uint32_t key = order_key(z);
            if (key > kept.floor_key && (key & path_mask) == (r.key & path_mask)) {
                const int b = (key >> shift) & 15;
                if (with_mass) sh->bins_f[b][threadIdx.x] += expf(z - zmax);
                sh->bins_i[b][threadIdx.x] += 1;
            }
        }
        cluster_bucket_totals(c);
        float mass[16];
        int count[16];
#pragma unroll
        for (int b = 0; b < 16; ++b) {
            mass[b] = sh->tot_f[b];
            count[b] = sh->tot_i[b];
        }
        // the tied elements at the floor are candidates too
        if (kept.floor_ties > 0 && (kept.floor_key & path_mask) == (r.key & path_mask)) {
            const int fb = (kept.floor_key >> shift) & 15;
#pragma unroll
            for (int b = 0; b < 16; ++b)
                if (b == fb) {
                    mass[b] += (float)kept.floor_ties * kept.floor_q;
                    count[b] += kept.floor_ties;
                }
        }
        if (level == 0) {
#pragma unroll
            for (int b = 15; b >= 0; --b) r.total_mass += mass[b];
            want_mass = fraction * r.total_mass;
        }
        // from the largest bucket down: the first one in which the target is crossed
        int pick = -1, last_nonempty = -1, last_count = 0, pick_count = 0;
        float last_mass = 0.f, pick_mass = 0.f;
        int cnt = r.above_count;
        float ms = r.above_mass;
#pragma unroll
        for (int b = 15; b >= 0; --b) {
            if (pick < 0 && count[b] > 0) {
                last_nonempty = b;
                last_count = count[b];
                last_mass = mass[b];
                const int c2 = cnt + count[b];
                const float m2 = ms + mass[b];
                const bool crossed = by_mass ? (inclusive ? m2 >= want_mass : m2 > want_mass)
                                             : c2 >= want_count;
                if (crossed) {
                    pick = b;
                    pick_count = count[b];
                    pick_mass = mass[b];
                } else {
                    cnt = c2;
                    ms = m2;
                }
            }
        }
        if (pick < 0) {
            // rounding left the target just beyond the end: the last candidate it is
            pick = last_nonempty < 0 ? 0 : last_nonempty;
            cnt -= last_count;
            ms -= last_mass;
            pick_count = last_count;
            pick_mass = last_mass;
        }
        r.above_count = cnt;
        r.above_mass = ms;
        r.key |= (uint32_t)pick << shift;
        if (few_enough > 0 && cnt + pick_count <= few_enough) {
            // the caller wants the candidates themselves, and they are few: every element at
            // or above the bucket's lowest key (r.key with the lower bits clear) is one
            r.ties = pick_count;
            r.few = true;
            return r;
        }
        if (level == 7) {
            r.ties = pick_count;
            r.q = pick_count > 0 ? pick_mass / (float)pick_count : 0.f;
        }
    }
    return r;
}

// Publish one integer per block (one block holds a value >= 0, the others -1) and
// return that value in every block (-1 if nobody had one).
__device__ int cluster_share_found(Cluster& c, int found) {
    SampleShared* sh = c.sh;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        sh->bins_f[k][threadIdx.x] = 0.f;
        sh->bins_i[k][threadIdx.x] = (k == 0 && threadIdx.x == 0) ? found + 1 : 0;
    }
    cluster_bucket_totals(c);
    return sh->tot_i[0] - 1;
}

// Token index of the `rank`-th (0-based, by index) element whose key equals `key`;
// every block returns it.
__device__ int nth_with_key(Cluster& c, const float* row, int lo, int hi, float inv_t,
                            uint32_t key, int rank) {
    SampleShared* sh = c.sh;
    const int n = hi - lo;
    const int per = (n + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int a = min(hi, lo + (int)threadIdx.x * per), b = min(hi, a + per);
    int mine = 0;
    for (int i = a; i < b; ++i) mine += order_key(row[i] * inv_t) == key;
#pragma unroll
    for (int k = 0; k < 16; ++k) {
        sh->bins_f[k][threadIdx.x] = 0.f;
        sh->bins_i[k][threadIdx.x] = k == 0 ? mine : 0;
    }
    sh->scan[threadIdx.x] = mine;
    cluster_bucket_totals(c);
    if (threadIdx.x == 0) {
        // matches in the blocks before this one (blocks are in index order), then in the
        // threads before each thread
        const int buf = (c.pass - 1) & 1;
        int run = 0;
        for (int k = 0; k < c.rank; ++k) run += c.first->xchg.i[buf][k][0];
        for (int t = 0; t < SAMPLE_THREADS; ++t) {
            const int v = sh->scan[t];
            sh->scan[t] = run;
            run += v;
        }
        sh->result = -1;
    }
    __syncthreads();
    const int before = sh->scan[threadIdx.x];
    if (rank >= before && rank < before + mine) {
        int seen = before;
        for (int i = a; i < b; ++i)
            if (order_key(row[i] * inv_t) == key) {
                if (seen == rank) { sh->result = i; break; }
                ++seen;
            }
    }
    __syncthreads();
    return cluster_share_found(c, sh->result);
}

// The top-k set as a list, when it is short: every block appends its elements with a key
// of at least `floor_key` to the first block's list; the first block sorts the list
// (descending z, ties by index: the order of the reference's sorted candidates), keeps
// `top_k` of them and does the rest as the reference does it, one candidate after the
// other: softmax, the shortest prefix whose mass reaches top_p, renormalisation, the draw
// (src/engine/sampler.rs:100-152).  Returns the token in the first block's first thread
// (-1 elsewhere); the caller shares it.
__device__ int sample_from_short_list(Cluster& c, const float* row, int lo, int hi, float inv_t,
                                      float zmax, uint32_t floor_key, int top_k, float top_p,
                                      float r, int fallback, float whole_mass = -1.f) {
    SampleShared* sh = c.sh;
    for (int i = lo + threadIdx.x; i < hi; i += SAMPLE_THREADS) {
        const float z = row[i] * inv_t;
        if (order_key(z) >= floor_key) {
            const int slot = atomicAdd(&c.first->list_n, 1);
            if (slot < SAMPLE_LIST) {
                c.first->list_z[slot] = z;
                c.first->list_i[slot] = i;
            }
        }
    }
    c.g.sync();
    int token = -1;
    if (c.rank == 0) {
        const int n = min(sh->list_n, SAMPLE_LIST);
        if ((int)threadIdx.x < n) {
            const float z = sh->list_z[threadIdx.x];
            const int idx = sh->list_i[threadIdx.x];
            int before = 0;
            for (int j = 0; j < n; ++j) {
                const float zj = sh->list_z[j];
                before += (zj > z) || (zj == z && sh->list_i[j] < idx);
            }
            sh->sorted_z[before] = z;
            sh->sorted_i[before] = idx;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            const int kept = min(n, top_k);
            float total = 0.f;
            for (int j = 0; j < kept; ++j) {
                sh->list_z[j] = expf(sh->sorted_z[j] - zmax);      // (the list's own maximum is zmax)
                total += sh->list_z[j];
            }
            // (without top-k the list is the head of the whole vocabulary, whose mass the
            // caller brings: the list reaches beyond the place where top_p is crossed)
            if (whole_mass >= 0.f) total = whole_mass;
            int cut = kept;
            float mass = total;           // of the candidates that stay
            if (top_p < 1.0f) {
                float cum = 0.f;
                mass = 0.f;
                for (int j = 0; j < kept; ++j) {
                    const float pj = sh->list_z[j] / total;
                    cum += pj;
                    mass += sh->list_z[j];
                    if (cum >= top_p) {
                        cut = j + 1;
                        break;
                    }
                }
            }
            token = kept > 0 ? sh->sorted_i[cut - 1] : fallback;
            float cum = 0.f;
            for (int j = 0; j < cut; ++j) {
                cum += sh->list_z[j] / mass;
                if (r < cum) {
                    token = sh->sorted_i[j];
                    break;
                }
            }
        }
    }
    return token;
}

__global__ void __cluster_dims__(SAMPLE_CLUSTER, 1, 1) __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(SampleArgs p) {
    extern __shared__ __align__(16) unsigned char sample_smem[];
    SampleShared* sh = reinterpret_cast<SampleShared*>(sample_smem);
    pdl_trigger();
    pdl_wait();
    Cluster c{cg::this_cluster(), sh, nullptr, 0, 0};
    c.rank = (int)c.g.block_rank();
    c.first = c.g.map_shared_rank(sh, 0);
    const int rowi = blockIdx.y;
    const float* row = p.logits + (size_t)rowi * p.stride;
    const int V = p.vocab;
    const int per_block = (V + SAMPLE_CLUSTER - 1) / SAMPLE_CLUSTER;
    const int lo = min(V, c.rank * per_block), hi = min(V, lo + per_block);
    const int which = p.rng_index ? p.rng_index[rowi] : rowi;
    const unsigned long long rng_before = p.temperature > 0.f ? p.rng[which] : 0ull;
    if (threadIdx.x == 0) sh->list_n = 0;
    c.g.sync();   // every block is running and has read the generator's state

    // ---- the maximum and its first index ----
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += SAMPLE_THREADS) {
        const float v = row[i];
        if (v > best) { best = v; best_i = i; }     // ascending i per thread: first maximum
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
    }
    if ((threadIdx.x & 31) == 0) {
        sh->warp_f[threadIdx.x >> 5] = best;
        sh->warp_i[threadIdx.x >> 5] = best_i;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SAMPLE_WARPS; ++w) {
            const float ov = sh->warp_f[w];
            const int oi = sh->warp_i[w];
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        c.first->xchg.f[c.pass & 1][c.rank][0] = best;
        c.first->xchg.i[c.pass & 1][c.rank][0] = best_i;
    }
    c.g.sync();
    {
        const int buf = c.pass & 1;
        best = c.first->xchg.f[buf][0][0];
        best_i = c.first->xchg.i[buf][0][0];
        for (int b = 1; b < SAMPLE_CLUSTER; ++b) {
            const float ov = c.first->xchg.f[buf][b][0];
            const int oi = c.first->xchg.i[buf][b][0];
            if (ov > best || (ov == best && oi < best_i)) { best = ov; best_i = oi; }
        }
        c.pass++;
    }
    if (p.temperature <= 0.f) {
        if (c.rank == 0 && threadIdx.x == 0) p.out[rowi] = best_i == 0x7fffffff ? 0 : best_i;
        c.g.sync();     // the first block's memory stays until every block has read it
        return;
    }
    // The reference divides by T; 1/T times z differs from that in the last bit at most,
    // and every pass uses the same product.
    const float inv_t = 1.0f / p.temperature;
    const float zmax = best * inv_t;
    unsigned long long x = rng_before;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    const float r = (float)(x >> 40) / 16777216.0f;
    if (c.rank == 0 && threadIdx.x == 0) p.rng[which] = x;

    const bool use_k = p.top_k > 0 && p.top_k < V;
    const bool use_p = p.top_p < 1.0f;
    int token;

    if (!use_k && !use_p) {
        // running sum by token index: blocks, then threads, own contiguous runs
        const int n = hi - lo;
        const int per = (n + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
        const int a = min(hi, lo + (int)threadIdx.x * per), b = min(hi, a + per);
        float mine = 0.f;
        for (int i = a; i < b; ++i) mine += expf(row[i] * inv_t - zmax);
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            sh->bins_f[k][threadIdx.x] = 0.f;
            sh->bins_i[k][threadIdx.x] = 0;
        }
        sh->scan_f[threadIdx.x] = mine;
        __syncthreads();
        if (threadIdx.x == 0) {
            float run = 0.f;      // this block's mass, threads in order
            for (int t = 0; t < SAMPLE_THREADS; ++t) run += sh->scan_f[t];
            sh->bins_f[0][0] = run;
        }
        cluster_bucket_totals(c);
        if (threadIdx.x == 0) {
            const int buf = (c.pass - 1) & 1;
            float acc = 0.f, all = 0.f;
            for (int k = 0; k < SAMPLE_CLUSTER; ++k) {
                if (k == c.rank) acc = all;
                all += c.first->xchg.f[buf][k][0];
            }
            sh->before_f = acc;
            sh->total_f = all;
            float run = acc;
            for (int t = 0; t < SAMPLE_THREADS; ++t) {
                const float v = sh->scan_f[t];
                sh->scan_f[t] = run;
                run += v;
            }
            sh->result = -1;
        }
        __syncthreads();
        const float target = r * sh->total_f;
        const float before = sh->scan_f[threadIdx.x];
        if (b > a && target >= before && target < before + mine) {
            float cum = before;
            int pick = b - 1;
            for (int i = a; i < b; ++i) {
                cum += expf(row[i] * inv_t - zmax);
                if (target < cum) { pick = i; break; }
            }
            sh->result = pick;
        }
        __syncthreads();
        token = cluster_share_found(c, sh->result);
        if (token < 0) token = V - 1;      // the reference's fallback: the last candidate
    } else {
        Kept kept{0u, 0, 0.f};
        bool listed = false;
        if (use_k) {
            // (the search for the k-th largest counts only: no masses are summed)
            // (and it stops as soon as the bucket it has come to, with everything above it,
            // fits the list: the list is sorted anyway)
            const Crossing k = find_crossing(c, row, lo, hi, inv_t, zmax, kept, false, p.top_k, 0.f,
                                             true, false, SAMPLE_LIST);
            if (k.above_count + k.ties <= SAMPLE_LIST) {
                listed = true;
                token = sample_from_short_list(c, row, lo, hi, inv_t, zmax, k.key, p.top_k, p.top_p,
                                               r, best_i);
                token = cluster_share_found(c, token);
                if (token < 0) token = best_i;
            } else {
                kept.floor_key = k.key;
                kept.floor_ties = max(0, min(k.ties, p.top_k - k.above_count));
                kept.floor_q = expf(key_value(k.key) - zmax);
            }
        }
        if (!use_k && use_p) {
            // the place where the mass reaches top_p, or, if the walk gets to a bucket that
            // fits the list with everything above it first, the head of the vocabulary as a list
            const Crossing q = find_crossing(c, row, lo, hi, inv_t, zmax, kept, true, 0, p.top_p,
                                             true, true, SAMPLE_LIST);
            if (q.few) {
                listed = true;
                token = sample_from_short_list(c, row, lo, hi, inv_t, zmax, q.key, SAMPLE_LIST,
                                               p.top_p, r, best_i, q.total_mass);
                token = cluster_share_found(c, token);
                if (token < 0) token = best_i;
            } else {
                const float want = p.top_p * q.total_mass;
                int need = q.ties;
                if (q.q > 0.f) need = max(1, min(q.ties, (int)ceilf((want - q.above_mass) / q.q)));
                kept.floor_key = q.key;
                kept.floor_ties = need;
                kept.floor_q = q.q;
            }
        }
        if (listed) {
            // (done above)
        } else {
        if (use_k && use_p) {
            const Crossing q = find_crossing(c, row, lo, hi, inv_t, zmax, kept, true, 0, p.top_p,
                                             true);
            const float want = p.top_p * q.total_mass;
            int need = q.ties;
            if (q.q > 0.f) need = max(1, min(q.ties, (int)ceilf((want - q.above_mass) / q.q)));
            kept.floor_key = q.key;
            kept.floor_ties = need;
            kept.floor_q = q.q;
        }
        // the draw lands on the first candidate whose running mass exceeds r x total
        const Crossing d = find_crossing(c, row, lo, hi, inv_t, zmax, kept, true, 0, r, false);
        const float target = r * d.total_mass;
        int rank = d.q > 0.f ? (int)floorf((target - d.above_mass) / d.q) : 0;
        rank = max(0, min(rank, d.ties - 1));
        token = nth_with_key(c, row, lo, hi, inv_t, d.key, rank);
        if (token < 0) token = best_i;
        }
    }
    if (c.rank == 0 && threadIdx.x == 0) p.out[rowi] = token;
    c.g.sync();         // the first block's memory stays until every block has read it
}

SIB_EXPORT int sib_sample_rows(const float* logits, long long stride, int rows, int vocab,
                               float temperature, int top_k, float top_p,
                               unsigned long long* rng, const int* rng_index, int* out,
                               void* stream) {
    if (rows == 0) return 0;
    SIB_REQUIRE(rows > 0 && rows < 65536 && vocab > 0 && stride >= vocab,
                "sample_rows: rows=%d vocab=%d", rows, vocab);
    SIB_REQUIRE(temperature <= 0.f || rng != nullptr, "sample_rows: sampling needs generator states");
    SIB_REQUIRE(top_k >= 0 && top_p > 0.f, "sample_rows: top_k=%d top_p=%f", top_k, top_p);
    SampleArgs p{logits, stride, vocab, temperature, top_k, top_p, rng, rng_index, out};
    const size_t smem = sizeof(SampleShared);
    cudaError_t e = cudaFuncSetAttribute(sample_rows_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
        sib_set_error("sample_rows: shared memory: %s", cudaGetErrorString(e));
        return (int)e;
    }
    e = sib_launch_chained(sample_rows_kernel, dim3(SAMPLE_CLUSTER, rows), dim3(SAMPLE_THREADS),
                           smem, (cudaStream_t)stream, p);
    if (e != cudaSuccess) {
        sib_set_error("sample_rows: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return sib_check_launch("sample_rows");
}
