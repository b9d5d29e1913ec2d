// mv_attention_decode_static: decode attention for callers that cannot allocate.
//
// This entry point has no counterpart in the reference engine; it exists for
// users of this library.
//
// Who needs it.  mv_attention_decode wants three pieces of scratch memory from
// its caller (partial sums of the key splits and a few counters).  Some callers
// have no way to get device memory at the moment they call: code that runs
// inside a region where the CUDA allocator must not be entered (a host callback,
// a library that was handed a fixed arena and nothing else, a runtime whose
// allocator belongs to another component and may not be called re-entrantly),
// or a plain C program that links this library without PyTorch and does not want
// to manage buffers.  For them the scratch lives inside the library itself, in a
// file-scope device array.  The caller still passes its inputs and its output.
//
// What it costs.  The array is part of the library image:
//   MV_STATIC_ATTN_MAX_TICKETS ints + MV_STATIC_ATTN_MAX_FLOATS floats  (about 4.1 MiB)
// on EVERY GPU that loads the library, from load until the process exits.
//
// Limits.  With splits > 1 a call needs  N * nkv * ceil((nh/nkv) / gt)  counters
// and  N * nh * splits * (hd + 2)  floats; with splits == 1 it needs no scratch
// at all and any N is taken (gt = 1, 2, 4 or 8: the
// smallest of these that is >= nh/nkv, at most 8).  A call that needs more than
// the array holds is refused: the function returns 2 and writes the two numbers
// into errbuf.  It never falls back to allocating.
//
// Rules of use.
//   * The first call on a device looks up the array's device address
//     (cudaGetSymbolAddress) and remembers it.  Make that first call with the
//     device current, before you begin any stream capture on that device, and
//     from one thread: the remembered address is written without a lock (two
//     threads that race there both write the same value).
//   * Every call uses the same array.  The function clears the counters on the
//     given stream before the kernel runs, so leftovers of an earlier call do no
//     harm; but two calls that overlap on the GPU (different streams, or the
//     same array reached from two processes' worth of threads) race on it and
//     give wrong results.  Order your calls on one stream, or with events.
//   * It calls no cudaMalloc, cudaFree or any other allocating routine.
//
// Arguments are those of mv_attention_decode without the three scratch
// pointers and without gt/head_tiles (worked out inside), plus errbuf: a buffer
// of errbuf_len bytes that receives a message when the return value is not 0
// (1 bad arguments, 2 too large for the built-in scratch, 3 a CUDA runtime call
// failed, 4 the launch failed).  dtype: 0 float32, 1 bfloat16.
#pragma once
#include <cuda_runtime.h>

#define MV_STATIC_ATTN_MAX_TICKETS 16384
#define MV_STATIC_ATTN_MAX_FLOATS (1 << 20)

extern "C" __attribute__((visibility("default"))) int mv_attention_decode_static(
    const void* q, const void* pool, long long page_stride, const int* page_table, int table_stride,
    int page_size, const int* positions, const int* seq_of, void* o, int dtype, int N, int nh, int nkv, int hd,
    float scale, int window, int splits, cudaStream_t stream, char* errbuf, int errbuf_len);
