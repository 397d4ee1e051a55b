// The phases of sib_decode_chain (decode_chain.cu), as its callers describe them.
#pragma once

#include "common.cuh"

#define SIB_CHAIN_MAX_PHASES 8

enum { SIB_CHAIN_PRODUCT = 0, SIB_CHAIN_NORM = 1 };
enum { SIB_CHAIN_EPI_NONE = 0, SIB_CHAIN_EPI_SOFTCAP = 1, SIB_CHAIN_EPI_GEGLU = 2, SIB_CHAIN_EPI_ROPE = 3 };

// One phase.  Pointers are device addresses; a field that a kind does not use is zero.
struct SibChainPhase {
    int kind;                 // SIB_CHAIN_PRODUCT or SIB_CHAIN_NORM
    int epi;                  // product: epilogue
    // ---- product: y[R, N] = epilogue(x[R, K] . w[N, K]^T), bfloat16 x and w ----
    const void* w;
    const void* x;
    void* y;                  // bfloat16, or 32-bit when out_f32 (plain and capped epilogue)
    int N, K, x_stride, y_stride, out_f32;
    float cap;
    // the rotating q|k|v product (SIB_CHAIN_EPI_ROPE): half-split pairs over the whole head,
    // k and v also written into the paged cache (k_pool null: nothing is stored)
    const int* row_pos;
    const int* row_seq;
    const int* seq_slot;
    const int* seq_end;
    const float* inv_freq;
    void* k_pool;
    void* v_pool;
    const int* page_table;
    int n_heads, n_kv, head_dim, max_pages, page_tokens, ring_tokens;
    // ---- norm: h[r] += post_gain ? rms(a[r]) * post_gain : a[r]; out[r] = rms(h[r]) * pre_gain.
    // Without a: out[r] = rms(h[rows ? rows[r] : r]) * pre_gain, h unchanged. ----
    const void* a;            // bfloat16 [R, hidden]
    const float* post_gain;
    float* h;                 // the 32-bit residual stream [R, hidden]
    const float* pre_gain;
    void* out;                // bfloat16 [R, hidden]
    const int* rows;
    float post_eps, pre_eps;
    int hidden, a_stride, out_stride;
};

SIB_EXPORT int sib_decode_chain(const SibChainPhase* phases, int n_phases, int R, int stages,
                                int* sync, void* stream);
SIB_EXPORT int sib_decode_chain_max_phases();
