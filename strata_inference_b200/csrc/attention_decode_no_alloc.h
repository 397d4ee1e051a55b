// sib_attention_decode_no_alloc: decode attention for hosts that cannot allocate.
//
// This entry point has no counterpart in the reference; it is an addition of
// this library.
//
// Who it is for.  sib_attention_decode cuts long key ranges into splits and needs
// a few megabytes of device memory for the splits' partial results, which its
// caller has to provide.  Some callers have nowhere to get that memory from at
// the moment of the call: a plain C host that links this library without an
// allocator of its own; a process that handed all device memory to its pools at
// start-up and keeps none back; a serving loop with a latency budget in which
// cudaMalloc is off limits because it may wait for the whole device.  For them
// the partial results live in an array that is part of the library's image.
//
// What it costs.  The array is 8 MiB (NO_ALLOC_SCRATCH_FLOATS 32-bit floats).
// Every GPU on which this library is loaded holds it from load until the process
// exits, whether or not this entry point is ever called.
//
// Limits.  The first NO_ALLOC_TICKET_SLOTS words of the array are ticket counters, one
// per (row, kv head) of a call; the partial results follow, rows * n_heads * splits *
// (head_dim + 2) floats with splits > 1 (sib_attention_decode_no_alloc_floats gives the
// sum).  A call whose rows * n_kv exceeds NO_ALLOC_TICKET_SLOTS, or whose sum exceeds
// NO_ALLOC_SCRATCH_FLOATS, is refused with an error (sib_last_error() says how much was
// asked for) and nothing is launched.  With splits == 1 the array is not used.
//
// Behaviour.  Arguments, result and arithmetic are those of sib_attention_decode
// without its `partial` and `tickets` arguments.  It calls no cudaMalloc, no cudaFree and no
// allocating library routine.  The first call on a device looks up the array's
// device address (cudaGetSymbolAddress, with that device current) and keeps it;
// make that first call on each device before any stream capture begins.  All
// calls share the one array, which keeps what the last call left in it.  The partial
// results need no initial value: every element that is read was written earlier in the
// same launch.  The ticket counters a launch uses have to be zero when it begins: each
// call clears them on its stream (a memset, no allocation) before it launches, so a
// launch that failed midway and left its counters non-zero does not spoil the next.
// The counters and the partial results never share an address, whatever the shapes of
// successive calls.  Two calls that overlap on the GPU (different streams, or several
// host threads) write over each other's partial results and tickets: run calls that
// use splits > 1 one after another on a device.
#pragma once

#include "common.cuh"

#define NO_ALLOC_SCRATCH_FLOATS (2u * 1024u * 1024u)
#define NO_ALLOC_TICKET_SLOTS 4096u

SIB_EXPORT int sib_attention_decode_no_alloc(
    const void* q, int q_stride, const void* k_pool, const void* v_pool, const int* page_table,
    int max_pages, int page_tokens, int ring_tokens, const int* row_pos, const int* row_seq,
    const int* seq_slot, void* out, int rows, int n_heads, int n_kv, int head_dim, float scale,
    float softcap, int window, int splits, void* stream);

// How many floats of the built-in array a call of this shape would use.
SIB_EXPORT long long sib_attention_decode_no_alloc_floats(int rows, int n_heads, int head_dim,
                                                          int splits);
