// Decode attention for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference; it exists for users of this library.
//
// Who needs it: code that runs where cudaMalloc is off limits — a plug-in inside a host
// application that owns the whole device heap and hands out fixed buffers only, a hard
// real-time loop that may not take the allocator's locks or its implicit synchronisation, or
// a process whose device memory is already taken up by weights and cache.  Such a
// caller can still provide the inputs and the output, but not the scratch memory that the
// split-range decode attention needs for its partial results.  Here that scratch lives in a
// fixed array inside the library.
//
// What it costs: the array is CRETIF_NOALLOC_SCRATCH_BYTES (4 MiB) of device memory on every
// GPU that loads the library, held until the process exits, whether or not this function is
// ever called.
//
// Limits: the call is refused (return value -1, nothing launched) when
//   B * nkv > CRETIF_NOALLOC_MAX_COUNTERS, or
//   B * nh * n_splits * (hd + 2) * 4 bytes exceed the array's float region,
// and otherwise takes what cretif_attn_decode_mma takes (bfloat16, head_dim a multiple of 16
// up to 128, 64-token cache blocks, n_splits <= 64).
//
// Sharing: all calls on a device use the same array.  Each call first clears the part that
// must start at zero (the range counters) on the given stream, so a call never sees what an
// earlier one left; but two calls whose kernels can overlap on the GPU (different streams
// without an ordering between them, or several host threads) race on the array and must be
// serialised by the caller.
//
// Set-up: the first call on a device looks up the array's device address
// (cudaGetSymbolAddress) with that device current.  Make that first call outside of any
// stream capture.
//
// It calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once

#define CRETIF_NOALLOC_SCRATCH_BYTES (4u << 20)
#define CRETIF_NOALLOC_MAX_COUNTERS 4096

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and result as cretif_attn_decode_mma, without the scratch pointers.
int cretif_attn_decode_noalloc(const void* q, int ldq, void* out, int ldo, const void* kc,
                               const void* vc, long long n_blocks, const int* table,
                               int table_stride, const int* tok_pos, const int* tok_seq,
                               const int* seq_slot, int nh, int nkv, int hd, float scale,
                               int window, int bt, int B, int n_splits, unsigned int* fault,
                               void* stream);

// Bytes of the fixed scratch array (for callers that want to check a shape beforehand).
unsigned int cretif_attn_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
