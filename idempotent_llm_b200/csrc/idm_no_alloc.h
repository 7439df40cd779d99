// An entry point that allocates nothing.  It has no counterpart in the reference.
//
// Who needs it.  The library's usual entry points take their scratch memory from the caller, and
// the Python side gets it from torch's allocator.  Some hosts cannot do that: a C or C++ process
// that loads this library by itself has no torch allocator to ask, and a serving process that has
// split the GPU's memory between weights and cache at start-up may forbid cudaMalloc afterwards,
// because it blocks the device while it runs and can fail once memory is fragmented.  Such a caller
// still owns its inputs and outputs; what it cannot supply is the scratch between the two kernels
// of the decode attention (the per-chunk partial results).
//
// What it is.  idm_attention_decode_static computes exactly what idm_attention_decode computes
// (attention of one query per sequence over that sequence's cached keys and values, see
// attention_decode.cu), with the partial results kept in an array that is part of the loaded
// library: IDM_NO_ALLOC_MAX_SCRATCH_FLOATS 32-bit floats (16 MiB).  Every GPU on which the library
// is loaded holds that array until the process exits.
//
// Limits and rules.
//  * 65536 + n_seqs * n_q * ceil(max_kv_len / 256) * (head_dim + 2) must not exceed
//    IDM_NO_ALLOC_MAX_SCRATCH_FLOATS; a larger request is refused with a message
//    (idm_last_error) and nothing is launched.
//  * The function calls no cudaMalloc, cudaFree or other allocating routine.
//  * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
//    that device current).  Make that first call outside any stream capture.
//  * All calls share the one array, which keeps what the last call left in it.  The partial results
//    need no clearing (each call writes every one it later reads); the small arrival counters
//    behind them must be zero when a call starts, which holds because the array starts as zeros
//    and every call sets its counters back before it ends -- also a call whose max_kv_len is smaller
//    than one of its kv_len: that sequence is then read only up to max_kv_len (rounded up to 256), a
//    wrong answer for a wrong call, but no chunk is waited for that the grid does not have.  Two calls
//    that overlap on the GPU, on different streams, race on the array: keep them on one stream or
//    order them with events.
//
// Arguments are those of idm_attention_decode without `scratch`:
//   q [n_seqs, n_q, hd] and out [n_seqs, n_q * hd] in the library's storage type; the cache entry's
//   k_pool / v_pool [pages, n_kv, 64, hd]; table [slots, table_stride] page numbers; ring (0, or the
//   ring length of a windowed entry); slots [n_seqs]; kv_len [n_seqs] lengths including the query's
//   own position; scale; window (0: none); the stream to launch on.  Returns 0, or 1 after
//   recording a message.
#pragma once

#include <cuda_runtime.h>

#define IDM_NO_ALLOC_MAX_SCRATCH_FLOATS (4 * 1024 * 1024)

extern "C" int idm_attention_decode_static(const void* q, void* out, void* k_pool, void* v_pool,
                                           const int* table, int table_stride, int ring, const int* slots,
                                           const int* kv_len, int n_seqs, int n_q, int n_kv, int hd,
                                           int max_kv_len, float scale, int window, cudaStream_t stream);
