// A chain of dependent few-row steps of decoding as ONE kernel: products y = x . W^T of
// at most 16 bfloat16 rows (with their epilogues) and the "norm, add, norm" steps between
// them, for everything that lies between two attention kernels of a decoder:
//
//     output projection | norm, add, norm | gate/up with gated GELU | down | norm, add, norm |
//     next layer's q|k|v with rotation and cache write
//
// or any other sequence of up to 8 such phases: the phases are data (a table in the kernel's
// parameters), and each names its own operands.
//
// One block per SM stays for the whole chain.  A ninth warp's first thread streams the
// weights of ALL phases, one after the other, through a ring of 16 KB tiles in shared
// memory (TMA loads over maps of this GPU's own memory, 128-byte swizzle, no multicast):
// weights depend on nothing, so the loader never waits for a phase to end, and the memory
// system stays busy while the eight computing warps wait for their inputs.  Those warps
// take a phase's units in turn (a unit: 16 x RG weight rows, all of k); activations come
// in chunks of 1 024 k, copied asynchronously into a double buffer; the products are
// mma.m16n8k16 with the weight rows as the A operand; a warp of a unit takes every KG-th
// 64-wide block of k (RG x KG = 8) and the KG partial sums are added in warp order.
// Between phases all blocks meet at a counter in global memory (the last block to leave
// the kernel puts the counters back to zero).  The first phase waits for the kernel
// before this one (programmatic dependent launch), the later ones for the counter.
//
// Arithmetic of the phases: the product and its epilogues as in linear_skinny.cu (soft
// cap; gated tanh-GELU over rows that come as 8 gate rows and their 8 up rows; rotation of
// q and k with cache write as in rope_cache.cu), "norm, add, norm" as in norm.cu
// (statistics, residual sum and gains in 32-bit).  Every wait is bounded; one that runs
// out leaves a code in the device's error word for this kernel and the block winds down.
// Plain counterparts: tests/plain_gemma2.py rms_norm(), gelu_tanh(), rope_neox(),
// x @ W.T.  Reference: src/model/layer.rs:1101-1192 (the order of a layer's steps).
#include "common.cuh"
#include "decode_chain.h"
#include "tma.cuh"

namespace {

constexpr int DC_BK = 64;                 // k per tile row: 128 bytes
constexpr int DC_STAGE = 16384;           // bytes per ring slot: 128 tile rows
constexpr int DC_WARPS = 8;
constexpr int DC_CONSUMERS = 32 * DC_WARPS;
constexpr int DC_THREADS = DC_CONSUMERS + 32;
constexpr int DC_XK = 1024;               // k of an activation chunk
constexpr int DC_XTILES = DC_XK / DC_BK;

struct alignas(64) Phase {
    CUtensorMap wmap;
    SibChainPhase d;
    int units, unit0, kg, ksteps;
    int k_tiled;           // the map is the 3-d one: one copy brings a whole ring slot
};

struct Chain {
    Phase ph[SIB_CHAIN_MAX_PHASES];
    int n_phases, R, stages, xbuf_bytes;
    int* sync;             // [0]: arrivals at the phase barriers, [1]: blocks that are done
    int* error_flag;
    unsigned long long* trace;   // measurements: [block][phase][4] nanosecond stamps, or null
};

__device__ __forceinline__ unsigned long long dc_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}

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
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
__device__ __forceinline__ void consumer_sync() {
    asm volatile("bar.sync 1, %0;\n" ::"n"(DC_CONSUMERS) : "memory");
}
__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float dc_gelu_tanh(float g) {
    const float c = 0.7978845608028654f;
    return 0.5f * g * (1.0f + tanhf(c * (g + 0.044715f * g * g * g)));
}

// Sum over the 256 computing threads; `scratch` holds 9 floats.
__device__ __forceinline__ float consumer_sum(float v, volatile float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    consumer_sync();
    if (lane == 0) scratch[warp] = v;
    consumer_sync();
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < DC_WARPS; ++w) t += scratch[w];     // in warp order, by every thread
    return t;
}

// The first unit of phase `ph` that block `cta` takes; it takes every `grid`-th after it.
__device__ __forceinline__ int first_unit(const Phase& ph, int cta, int grid) {
    int u = (cta - ph.unit0) % grid;
    return u < 0 ? u + grid : u;
}

// Where the two 8-row halves of a warp's 16 weight rows start.
__device__ __forceinline__ void unit_rows(const SibChainPhase& d, int rg_count, int unit, int rg,
                                          int& row_a, int& row_b) {
    if (d.epi == SIB_CHAIN_EPI_ROPE) {
        // 8 rows of a head's first half and the 8 rows half a head further on
        const int per_head = d.head_dim / (16 * rg_count);
        const int head = unit / per_head, i = unit % per_head;
        row_a = head * d.head_dim + 8 * rg_count * i + 8 * rg;
        row_b = row_a + d.head_dim / 2;
    } else {
        row_a = unit * 16 * rg_count + 16 * rg;
        row_b = row_a + 8;
    }
}

template <int NT>
__device__ __forceinline__ void product_epilogue(const SibChainPhase& d, int R, int row_a, int row_b,
                                                 int lane, float (&acc)[NT][4]) {
    const int g = lane >> 2, t = lane & 3;
    const int na = row_a + g, nb = row_b + g;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int r0 = 8 * j + 2 * t;
        if (d.epi == SIB_CHAIN_EPI_GEGLU) {
            // rows g (gate) and g + 8 (up) of a 16-row group make one output column
            __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(d.y);
            const int n_out = (row_a / 16) * 8 + g;
            if (nb < d.N) {
                if (r0 < R)
                    y[(size_t)r0 * d.y_stride + n_out] =
                        __float2bfloat16_rn(dc_gelu_tanh(acc[j][0]) * acc[j][2]);
                if (r0 + 1 < R)
                    y[(size_t)(r0 + 1) * d.y_stride + n_out] =
                        __float2bfloat16_rn(dc_gelu_tanh(acc[j][1]) * acc[j][3]);
            }
        } else if (d.epi == SIB_CHAIN_EPI_ROPE) {
            __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(d.y);
            const int hd = d.head_dim;
            const int head = na / hd, dim = na % hd;
            const bool rotates = head < d.n_heads + d.n_kv;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int r = r0 + e;
                if (r >= R || nb >= d.N) continue;
                const int pos = d.row_pos[r];
                float oa = acc[j][e], ob = acc[j][2 + e];
                if (rotates) {
                    const float ang = (float)pos * d.inv_freq[dim];
                    const float c = cosf(ang), sn = sinf(ang);
                    const float ia = oa, ib = ob;
                    oa = ia * c - ib * sn;
                    ob = ia * sn + ib * c;
                }
                y[(size_t)r * d.y_stride + na] = __float2bfloat16_rn(oa);
                y[(size_t)r * d.y_stride + nb] = __float2bfloat16_rn(ob);
                if (head >= d.n_heads && d.k_pool) {
                    const int b = d.row_seq[r];
                    int cell = pos;
                    bool keep = true;
                    if (d.ring_tokens > 0) {
                        keep = pos >= d.seq_end[b] - d.ring_tokens;
                        cell = pos % d.ring_tokens;
                    }
                    if (keep) {
                        const int page = d.page_table[(size_t)d.seq_slot[b] * d.max_pages +
                                                      cell / d.page_tokens];
                        const bool is_k = head < d.n_heads + d.n_kv;
                        const int kvh = head - d.n_heads - (is_k ? 0 : d.n_kv);
                        __nv_bfloat16* dst =
                            reinterpret_cast<__nv_bfloat16*>(is_k ? d.k_pool : d.v_pool) +
                            (((size_t)page * d.n_kv + kvh) * d.page_tokens + cell % d.page_tokens) * hd;
                        dst[dim] = __float2bfloat16_rn(oa);
                        dst[dim + hd / 2] = __float2bfloat16_rn(ob);
                    }
                }
            }
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                float o = acc[j][c];
                if (d.epi == SIB_CHAIN_EPI_SOFTCAP) o = d.cap * tanhf(o / d.cap);
                const int n = c >= 2 ? nb : na, r = r0 + (c & 1);
                if (n < d.N && r < R) {
                    if (d.out_f32) reinterpret_cast<float*>(d.y)[(size_t)r * d.y_stride + n] = o;
                    else reinterpret_cast<__nv_bfloat16*>(d.y)[(size_t)r * d.y_stride + n] =
                        __float2bfloat16_rn(o);
                }
            }
        }
    }
}

// h[r] += post_gain ? rms(a[r]) * post_gain : a[r];  out[r] = rms(h[r]) * pre_gain (if given).
// Without `a`: out[r] = rms(h[rows ? rows[r] : r]) * pre_gain and h stays as it is.
__device__ void norm_unit(const SibChainPhase& d, int r, float* row, volatile float* scratch) {
    const int H = d.hidden;
    const int src_row = (!d.a && d.rows) ? d.rows[r] : r;
    float* h = d.h + (size_t)src_row * H;
    float ss2 = 0.f;
    if (d.a) {
        const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(d.a) + (size_t)r * d.a_stride;
        float ss = 0.f;
        for (int c = threadIdx.x; c < H; c += DC_CONSUMERS) {
            const float v = __bfloat162float(__ldcg(a + c));     // written by other blocks
            row[c] = v;
            ss += v * v;
        }
        float inv = 1.f;
        if (d.post_gain) {
            ss = consumer_sum(ss, scratch);
            inv = 1.0f / sqrtf(ss / (float)H + d.post_eps);
        }
        for (int c = threadIdx.x; c < H; c += DC_CONSUMERS) {     // each thread its own columns
            const float add = d.post_gain ? row[c] * inv * d.post_gain[c] : row[c];
            const float v = __ldcg(h + c) + add;
            h[c] = v;
            row[c] = v;
            ss2 += v * v;
        }
    } else {
        for (int c = threadIdx.x; c < H; c += DC_CONSUMERS) {
            const float v = __ldcg(h + c);
            row[c] = v;
            ss2 += v * v;
        }
    }
    if (!d.pre_gain) return;
    ss2 = consumer_sum(ss2, scratch);
    const float inv2 = 1.0f / sqrtf(ss2 / (float)H + d.pre_eps);
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(d.out) + (size_t)r * d.out_stride;
    for (int c = threadIdx.x; c < H; c += DC_CONSUMERS)
        out[c] = __float2bfloat16_rn(row[c] * inv2 * d.pre_gain[c]);
}

template <int NT>
__global__ void __launch_bounds__(DC_THREADS, 1)
decode_chain_kernel(const __grid_constant__ Chain ch) {
    extern __shared__ uint8_t dc_raw[];
    const uint32_t raw = sib_smem_u32(dc_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* basep = dc_raw + (base - raw);
    constexpr int ROWS = NT * 8;
    const int stages = ch.stages;
    // ring of weight tiles | two activation chunks (or one row of a norm) | partial sums of
    // the warps | barriers
    const uint32_t ring = base;
    const uint32_t xbuf = ring + stages * DC_STAGE;
    const uint32_t red = xbuf + ch.xbuf_bytes;
    uint8_t* after = basep + stages * DC_STAGE + ch.xbuf_bytes + DC_WARPS * NT * 32 * 16;
    uint64_t* full = reinterpret_cast<uint64_t*>(after);
    uint64_t* empty = full + stages;
    volatile float* scratch = reinterpret_cast<volatile float*>(empty + stages);   // 16 floats
    volatile int* failed = reinterpret_cast<volatile int*>(const_cast<float*>(scratch) + 16);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta = blockIdx.x, grid = gridDim.x;

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            sib_mbar_init(&full[s], 1);
            sib_mbar_init(&empty[s], DC_WARPS);
        }
        *failed = 0;
        sib_mbar_init_fence();
    }
    __syncthreads();

    if (warp == DC_WARPS) {
        // ---- the loader: every phase's weights, one tile after the other ----
        if (lane == 0) {
            int i = 0;      // tiles issued so far
            for (int p = 0; p < ch.n_phases && !*failed; ++p) {
                const Phase& ph = ch.ph[p];
                if (ph.d.kind != SIB_CHAIN_PRODUCT) continue;
                const int kg = ph.kg, rg_count = DC_WARPS / kg;
                const bool rope = ph.d.epi == SIB_CHAIN_EPI_ROPE;
                const int sub = 16 * rg_count * 128;     // bytes of one 64-wide block of k
                for (int u = first_unit(ph, cta, grid); u < ph.units && !*failed; u += grid) {
                    int row_a, row_b;
                    unit_rows(ph.d, rg_count, u, 0, row_a, row_b);
                    for (int step = 0; step < ph.ksteps; ++step, ++i) {
                        const int s = i % stages;
                        if (i >= stages && !sib_mbar_wait(&empty[s], ((i / stages) - 1) & 1)) {
                            *failed = 1;
                            break;
                        }
                        sib_mbar_arrive_expect_tx(&full[s], DC_STAGE);
                        uint8_t* dst = basep + s * DC_STAGE;
                        // a slot holds [block of k][row][64]; the rotating product's two runs
                        // of rows each fill half a slot
                        if (ph.k_tiled) {
                            sib_tma_load_3d(dst, &ph.wmap, &full[s], 0, row_a, step * kg);
                            if (rope)
                                sib_tma_load_3d(dst + DC_STAGE / 2, &ph.wmap, &full[s], 0, row_b, step * kg);
                        } else {
                            for (int q = 0; q < kg; ++q) {
                                const int k = (step * kg + q) * DC_BK;
                                if (rope) {
                                    sib_tma_load_2d(dst + q * (sub / 2), &ph.wmap, &full[s], k, row_a);
                                    sib_tma_load_2d(dst + DC_STAGE / 2 + q * (sub / 2), &ph.wmap, &full[s],
                                                    k, row_b);
                                } else {
                                    sib_tma_load_2d(dst + q * sub, &ph.wmap, &full[s], k, row_a);
                                }
                            }
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else {
        // ---- the eight computing warps ----
        const int g = lane >> 2, t = lane & 3;
        const uint32_t c0 = (uint32_t)((2 * t) ^ g) << 4, c1 = (uint32_t)((2 * t + 1) ^ g) << 4;
        const uint4 zero = make_uint4(0, 0, 0, 0);
        int i = 0;          // tiles taken so far (the loader's count)
        pdl_wait();         // the first phase reads what the kernel before this one wrote
        for (int p = 0; p < ch.n_phases; ++p) {
            const Phase& ph = ch.ph[p];
            const SibChainPhase& d = ph.d;
            if (p > 0) {
                // every block has finished phase p - 1
                if (threadIdx.x == 0 && !*failed) {
                    const int want = p * grid;
                    bool ok = false;
                    for (uint32_t spin = 0; spin < SIB_WAIT_LIMIT; ++spin)
                        if (ld_acquire(ch.sync) >= want) { ok = true; break; }
                    if (!ok) *failed = 3;
                }
                consumer_sync();
            }
            // (after a failure the warps still walk through every phase, without waiting or
            // writing, so that the barriers between them keep matching)
            unsigned long long* tr = ch.trace ? ch.trace + ((size_t)cta * SIB_CHAIN_MAX_PHASES + p) * 4
                                              : nullptr;
            if (tr && threadIdx.x == 0) tr[0] = dc_now();       // the phase is open
            if (d.kind == SIB_CHAIN_NORM) {
                for (int u = first_unit(ph, cta, grid); u < ph.units; u += grid) {
                    norm_unit(d, u, reinterpret_cast<float*>(basep + stages * DC_STAGE), scratch);
                    consumer_sync();      // the row buffer may be overwritten
                }
            } else {
                const int kg_count = ph.kg, rg_count = DC_WARPS / kg_count;
                const int rg = warp / kg_count, kg = warp % kg_count;
                const bool rope = d.epi == SIB_CHAIN_EPI_ROPE;
                const uint32_t sub = 16 * rg_count * 128;
                const uint32_t wa_off = rope ? kg * (sub / 2) + (8 * rg + g) * 128
                                             : kg * sub + (16 * rg + g) * 128;
                const uint32_t wb_off = rope ? DC_STAGE / 2 + kg * (sub / 2) + (8 * rg + g) * 128
                                             : kg * sub + (16 * rg + 8 + g) * 128;
                const int steps_per_chunk = DC_XTILES / kg_count;
                const int n_chunks = (ph.ksteps + steps_per_chunk - 1) / steps_per_chunk;
                const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(d.x);
                const uint32_t chunk_bytes = DC_XTILES * ROWS * 128;
                // the activation chunk that starts at k0, into buffer `b` (asynchronous copies)
                auto fetch = [&](int b, int k0) {
                    const uint32_t dst0 = xbuf + b * chunk_bytes;
                    for (int idx = threadIdx.x; idx < DC_XTILES * ROWS * 8; idx += DC_CONSUMERS) {
                        const int c = idx & 7, r = (idx >> 3) % ROWS, kt = (idx >> 3) / ROWS;
                        const int k = k0 + kt * DC_BK + c * 8;
                        const uint32_t dst = dst0 + (kt * ROWS + r) * 128 + ((c ^ (r & 7)) << 4);
                        if (r < ch.R && k < d.K) cp_async16(dst, x + (size_t)r * d.x_stride + k);
                        else sts128(dst, zero);
                    }
                    cp_async_commit();
                };
                const int u_first = first_unit(ph, cta, grid);
                int seq = 0;        // chunks taken in this phase
                if (u_first < ph.units) fetch(0, 0);
                for (int u = u_first; u < ph.units; u += grid) {
                    float acc[NT][4];
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int c = 0; c < 4; ++c) acc[j][c] = 0.f;
                    for (int q = 0; q < n_chunks; ++q, ++seq) {
                        // the chunk after this one (of this unit or the first of the next unit)
                        const bool more = q + 1 < n_chunks || u + grid < ph.units;
                        if (more) fetch((seq + 1) & 1, q + 1 < n_chunks ? (q + 1) * DC_XK : 0);
                        if (more) cp_async_wait<1>(); else cp_async_wait<0>();
                        consumer_sync();
                        if (tr && threadIdx.x == 0 && seq == 0) tr[1] = dc_now();   // first activations
                        const uint32_t xb = xbuf + (seq & 1) * chunk_bytes;
                        const int step_end = min(ph.ksteps, (q + 1) * steps_per_chunk);
                        for (int step = q * steps_per_chunk; step < step_end; ++step, ++i) {
                            const int s = i % stages;
                            if (*failed) continue;
                            if (!sib_mbar_wait(&full[s], (i / stages) & 1)) {
                                *failed = 2;
                                continue;
                            }
                            const uint32_t tile = ring + s * DC_STAGE;
                            const uint4 wa0 = lds128(tile + wa_off + c0), wa1 = lds128(tile + wa_off + c1);
                            const uint4 wb0 = lds128(tile + wb_off + c0), wb1 = lds128(tile + wb_off + c1);
                            __syncwarp();
                            if (lane == 0) sib_mbar_arrive(&empty[s]);
                            const int kt = (step - q * steps_per_chunk) * kg_count + kg;
#pragma unroll
                            for (int j = 0; j < NT; ++j) {
                                const uint32_t xr = xb + (kt * ROWS + 8 * j + g) * 128;
                                const uint4 x0 = lds128(xr + c0), x1 = lds128(xr + c1);
                                mma_16816(acc[j], wa0.x, wb0.x, wa0.y, wb0.y, x0.x, x0.y);
                                mma_16816(acc[j], wa0.z, wb0.z, wa0.w, wb0.w, x0.z, x0.w);
                                mma_16816(acc[j], wa1.x, wb1.x, wa1.y, wb1.y, x1.x, x1.y);
                                mma_16816(acc[j], wa1.z, wb1.z, wa1.w, wb1.w, x1.z, x1.w);
                            }
                        }
                        consumer_sync();      // every warp is done with this chunk's buffer
                    }
                    // the KG warps of a run of rows add their sums in warp order
                    if (kg_count > 1) {
#pragma unroll
                        for (int j = 0; j < NT; ++j)
                            sts128(red + ((warp * NT + j) * 32 + lane) * 16,
                                   make_uint4(__float_as_uint(acc[j][0]), __float_as_uint(acc[j][1]),
                                              __float_as_uint(acc[j][2]), __float_as_uint(acc[j][3])));
                        consumer_sync();
                        if (kg == 0) {
                            for (int o = 1; o < kg_count; ++o) {
#pragma unroll
                                for (int j = 0; j < NT; ++j) {
                                    const uint4 v = lds128(red + (((warp + o) * NT + j) * 32 + lane) * 16);
                                    acc[j][0] += __uint_as_float(v.x);
                                    acc[j][1] += __uint_as_float(v.y);
                                    acc[j][2] += __uint_as_float(v.z);
                                    acc[j][3] += __uint_as_float(v.w);
                                }
                            }
                        }
                    }
                    if (kg == 0 && !*failed) {
                        int row_a, row_b;
                        unit_rows(d, rg_count, u, rg, row_a, row_b);
                        product_epilogue<NT>(d, ch.R, row_a, row_b, lane, acc);
                    }
                    if (kg_count > 1) consumer_sync();      // the partial sums may be overwritten
                }
            }
            if (tr && threadIdx.x == 0) tr[2] = dc_now();           // this block's units are done
            if (p + 1 < ch.n_phases) {
                __threadfence();
                consumer_sync();
                if (threadIdx.x == 0) atomicAdd(ch.sync, 1);
            }
            if (tr && threadIdx.x == 0) tr[3] = dc_now();
        }
        __syncwarp();
    }

    __syncthreads();
    if (threadIdx.x == 0) {
        if (*failed) atomicExch(ch.error_flag, *failed);
        __threadfence();
        // the last block to leave puts the counters back for the next launch
        if (atomicAdd(ch.sync + 1, 1) == grid - 1) {
            ch.sync[0] = 0;
            ch.sync[1] = 0;
            __threadfence();
        }
    }
}

int g_dc_sm_count[64] = {};
unsigned long long* g_dc_trace = nullptr;
int g_dc_force_rg = 0;      // experiments: rows of weight a unit takes are 16 x this (0: chosen)

// Rows of weight a unit takes (16 x RG, RG in {8, 4, 2, 1}): what fills the blocks best.
int choose_row_groups(const SibChainPhase& d, int grid) {
    int best = 0;
    double best_fill = -1.0;
    if (g_dc_force_rg > 0 &&
        !(d.epi == SIB_CHAIN_EPI_ROPE && (d.head_dim / 2) % (8 * g_dc_force_rg) != 0))
        return g_dc_force_rg;
    for (int rg = 8; rg >= 1; rg /= 2) {
        if (d.epi == SIB_CHAIN_EPI_ROPE && (d.head_dim / 2) % (8 * rg) != 0) continue;
        const int units = (d.N + 16 * rg - 1) / (16 * rg);
        const int waves = (units + grid - 1) / grid;
        const double fill = (double)units / ((double)waves * grid);
        if (fill > best_fill + 0.03) {     // larger runs of rows unless smaller ones fill better
            best_fill = fill;
            best = rg;
        }
    }
    return best;
}

}  // namespace

SIB_EXPORT int sib_decode_chain_max_phases() { return SIB_CHAIN_MAX_PHASES; }

// For measurements: later launches write, per block and phase, four %globaltimer stamps (the
// phase opened, the first activations arrived, the block's units were done, it arrived at
// the phase's end) into `buffer` (blocks x 8 x 4 64-bit words on the device; null: stop).
SIB_EXPORT void sib_decode_chain_trace(void* buffer) { g_dc_trace = (unsigned long long*)buffer; }

// For measurements: every product takes units of 16 x rg weight rows (rg 1, 2, 4 or 8; 0
// gives the choice back to the launcher).
SIB_EXPORT void sib_decode_chain_force_row_groups(int rg) {
    g_dc_force_rg = (rg == 1 || rg == 2 || rg == 4 || rg == 8) ? rg : 0;
}

// `sync`: two int32 counters in device memory, zero before the first launch (every launch
// leaves them zero).  `stages`: ring slots of 16 KB (0: as many as fit, at most 8).
SIB_EXPORT int sib_decode_chain(const SibChainPhase* phases, int n_phases, int R, int stages,
                                int* sync, void* stream) {
    SIB_REQUIRE(n_phases >= 1 && n_phases <= SIB_CHAIN_MAX_PHASES,
                "decode_chain: %d phases; 1 to %d", n_phases, SIB_CHAIN_MAX_PHASES);
    SIB_REQUIRE(R >= 1 && R <= 16, "decode_chain: %d rows; 1 to 16", R);
    SIB_REQUIRE(sync != nullptr && stages >= 0 && stages <= 12, "decode_chain: counters or stages");
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    SIB_REQUIRE(e == cudaSuccess && dev >= 0 && dev < 64, "decode_chain: no current device");
    if (!g_dc_sm_count[dev]) {
        e = cudaDeviceGetAttribute(&g_dc_sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
        SIB_REQUIRE(e == cudaSuccess && g_dc_sm_count[dev] > 0, "decode_chain: %s",
                    cudaGetErrorString(e));
    }
    const int grid = g_dc_sm_count[dev];
    int* error_flag = sib_error_word(SIB_ERR_DECODE_CHAIN);
    if (!error_flag) return -1;

    static thread_local Chain ch;
    ch.n_phases = n_phases;
    ch.R = R;
    ch.sync = sync;
    ch.error_flag = error_flag;
    ch.trace = g_dc_trace;
    const int NT = R <= 8 ? 1 : 2;
    int unit0 = 0, max_hidden = 0;
    for (int p = 0; p < n_phases; ++p) {
        Phase& ph = ch.ph[p];
        ph.d = phases[p];
        const SibChainPhase& d = ph.d;
        ph.unit0 = unit0;
        if (d.kind == SIB_CHAIN_NORM) {
            SIB_REQUIRE(d.h && d.hidden > 0 && (d.a || d.pre_gain) && (!d.pre_gain || d.out),
                        "decode_chain: phase %d: incomplete norm step", p);
            ph.units = R;
            ph.kg = 1;
            ph.ksteps = 0;
            ph.k_tiled = 0;
            if (d.hidden > max_hidden) max_hidden = d.hidden;
        } else if (d.kind == SIB_CHAIN_PRODUCT) {
            SIB_REQUIRE(d.w && d.x && d.y && d.N > 0 && d.K > 0 && d.K % 8 == 0 && d.x_stride % 8 == 0 &&
                            ((uintptr_t)d.w % 16) == 0 && ((uintptr_t)d.x % 16) == 0,
                        "decode_chain: phase %d: N=%d K=%d x_stride=%d; K and the row stride must "
                        "be multiples of 8 and the operands 16-byte aligned", p, d.N, d.K, d.x_stride);
            SIB_REQUIRE(d.epi >= SIB_CHAIN_EPI_NONE && d.epi <= SIB_CHAIN_EPI_ROPE,
                        "decode_chain: phase %d: unknown epilogue %d", p, d.epi);
            SIB_REQUIRE(d.epi != SIB_CHAIN_EPI_GEGLU || d.N % 16 == 0,
                        "decode_chain: phase %d: the gated epilogue needs N (%d) in groups of 16", p, d.N);
            SIB_REQUIRE(d.epi != SIB_CHAIN_EPI_SOFTCAP || d.cap > 0.f,
                        "decode_chain: phase %d: soft cap must be positive", p);
            SIB_REQUIRE(!d.out_f32 || d.epi == SIB_CHAIN_EPI_NONE || d.epi == SIB_CHAIN_EPI_SOFTCAP,
                        "decode_chain: phase %d: 32-bit outputs go with the plain and the capped "
                        "epilogue only", p);
            if (d.epi == SIB_CHAIN_EPI_ROPE) {
                SIB_REQUIRE(d.head_dim > 0 && d.head_dim % 16 == 0 && d.n_heads > 0 && d.n_kv >= 0 &&
                                d.N == (d.n_heads + 2 * d.n_kv) * d.head_dim && d.row_pos && d.inv_freq,
                            "decode_chain: phase %d: the rotating product needs heads=%d kv=%d "
                            "head_dim=%d (a multiple of 16) that make up N=%d", p, d.n_heads, d.n_kv,
                            d.head_dim, d.N);
                SIB_REQUIRE(d.n_kv == 0 || !d.k_pool ||
                                (d.v_pool && d.page_table && d.row_seq && d.seq_slot && d.seq_end &&
                                 d.page_tokens > 0 && d.max_pages > 0 && d.ring_tokens >= 0 &&
                                 (d.ring_tokens == 0 || d.ring_tokens % d.page_tokens == 0)),
                            "decode_chain: phase %d: incomplete cache description", p);
            }
            const int rg = choose_row_groups(d, grid);
            SIB_REQUIRE(rg > 0, "decode_chain: phase %d: head_dim %d cannot be tiled", p, d.head_dim);
            ph.kg = DC_WARPS / rg;
            ph.units = (d.N + 16 * rg - 1) / (16 * rg);
            ph.ksteps = (d.K + ph.kg * DC_BK - 1) / (ph.kg * DC_BK);
            const int box_rows = d.epi == SIB_CHAIN_EPI_ROPE ? 8 * rg : 16 * rg;
            ph.k_tiled = d.K % DC_BK == 0 && ph.kg > 1;
            if (ph.k_tiled) {
                if (sib_make_bf16_map_k_tiles(&ph.wmap, d.w, d.N, d.K, d.K, box_rows, ph.kg,
                                              "decode_chain")) return -1;
            } else if (sib_make_bf16_map(&ph.wmap, d.w, d.N, d.K, d.K, box_rows, "decode_chain")) {
                return -1;
            }
        } else {
            SIB_REQUIRE(false, "decode_chain: phase %d: unknown kind %d", p, d.kind);
        }
        unit0 += ph.units;
    }
    ch.xbuf_bytes = 2 * DC_XTILES * NT * 8 * 128;
    if (max_hidden * 4 > ch.xbuf_bytes) ch.xbuf_bytes = (max_hidden * 4 + 1023) / 1024 * 1024;
    const size_t fixed = 1024 + (size_t)ch.xbuf_bytes + DC_WARPS * NT * 32 * 16 + 12 * 16 + 128;
    int st = stages > 0 ? stages : 8;
    while (st > 2 && fixed + (size_t)st * DC_STAGE > 200 * 1024) --st;
    ch.stages = st;
    const size_t smem = fixed + (size_t)st * DC_STAGE;
    SIB_REQUIRE(smem <= 227 * 1024, "decode_chain: %zu bytes of shared memory a block", smem);

    auto kernel = NT == 1 ? decode_chain_kernel<1> : decode_chain_kernel<2>;
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) {
        sib_set_error("decode_chain: shared memory (%zu bytes): %s", smem, cudaGetErrorString(e));
        return (int)e;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(DC_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = sib_chained_launches() ? 1 : 0;
    sib_same_carveout(kernel);
    e = cudaLaunchKernelEx(&cfg, kernel, ch);
    if (e != cudaSuccess) {
        sib_set_error("decode_chain: launch failed: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return sib_check_launch("decode_chain");
}
