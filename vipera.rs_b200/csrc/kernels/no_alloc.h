// An entry point for callers that must not allocate device memory.
//
// This declaration has no counterpart in the reference: vipera.rs's device code allocates
// its buffers through its own Device wrapper and has no such variant.
//
// Who needs it.  Some programs that link this library cannot call cudaMalloc (or anything
// that calls it for them) at the moment they need a greedy token: code that runs inside a
// region where allocation is forbidden because it would synchronise the device or break a
// latency bound (a real-time control loop, a callback driven by another runtime that owns
// the memory pool), or a host that has handed all device memory to its own allocator and
// allows none on the side.  The ordinary argmax of this library, vipera_argmax, takes a
// scratch buffer from its caller, who usually gets it from an allocator.  The variant below
// brings its scratch with it instead.
//
// vipera_argmax_static(logits, rows, vocab, tokens, status, stream)
//   tokens[r] = index of the largest finite value of row r of `logits` ([rows, vocab]
//   float32, row-major), ties to the lowest index; status[r] (optional, may be null) is 0,
//   or 1 when the row holds no finite value.  All pointers are device pointers supplied by
//   the caller.  Returns 0, a negative code of this library (-2: more rows than
//   VIPERA_ARGMAX_STATIC_MAX_ROWS, or a vocabulary below 1; -3: a null pointer), or a
//   positive cudaError_t.
//
//   Its scratch (a value and an index for each of 32 slices of every row) is a file-scope
//   `static __device__` array of 64 * VIPERA_ARGMAX_STATIC_MAX_ROWS 32-bit words (256 KiB),
//   which every GPU that loads the library holds until the process ends.  The entry point
//   calls no cudaMalloc, cudaFree or allocating library routine.
//
//   The first call on a device looks up the array's device address (cudaGetSymbolAddress,
//   with that device current) and keeps it; make that first call outside any stream capture.
//   The kept address is written without a lock: two host threads that both make the first
//   call on a device both look it up and both store the same value, which is harmless, but
//   a program that wants no such overlap makes one call per device before it starts its threads.
//
//   All calls share the one array.  Every word a call reads was written earlier in the same
//   call, so nothing has to be cleared and what an earlier call left behind is never seen;
//   but two calls that overlap on the GPU (different streams, or the same call replayed
//   concurrently) write the same words and race.  Run them one after another.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define VIPERA_ARGMAX_STATIC_MAX_ROWS 1024

int vipera_argmax_static(const float* logits, int rows, int vocab, int* tokens, int* status, void* stream);

#ifdef __cplusplus
}
#endif
