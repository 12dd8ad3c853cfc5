// Allocation-free residual selection.  This entry point has no counterpart in the reference
// project; it exists for callers of this library that are not allowed to allocate device memory.
//
// Who cannot allocate: code running while a CUDA stream is being captured into a graph, code
// inside a framework's allocator-managed region that must not grow the pool (for example a
// memory-budgeted training step whose peak is planned ahead of time), and embedders that hand
// this library a fixed arena and forbid cudaMalloc/cudaFree because those calls synchronise the
// whole device.  The regular entry point (sb_residual_topk) needs a histogram and a few counters
// that its caller allocates per call; here that scratch is a file-scope device array inside the
// library, so the caller passes only inputs and outputs.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

// Largest number of row chunks one call may select over; the built-in scratch is sized for it
// (SB_NOALLOC_MAX_CHUNKS * 32768 four-byte histogram bins plus 8 ints per chunk, about 2 MB,
// resident on every GPU that loads the library until the process exits).
#define SB_NOALLOC_MAX_CHUNKS 16

// Number of (index, value) pairs a call with these arguments writes, or -1 for invalid arguments.
// Every full chunk of `chunk_rows` rows contributes `quota_per_chunk` entries; a short last chunk
// contributes round(quota_per_chunk * its_rows / chunk_rows), at least 1.
long long sb_residual_topk_noalloc_count(int rows, int chunk_rows, int quota_per_chunk);

// Exact per-chunk top-k by magnitude of the residual X - C Q^T, same semantics and output format
// as sb_residual_topk (bf16 inputs x [rows, n] with leading dimension ldx, c [rows, r], q [n, r];
// idx32 or idx64 (exactly one non-NULL) and val sized by sb_residual_topk_noalloc_count; val is
// bf16 when bits == 0 and int8 codes when bits is 8 or 4; scale is one fp32 on the device).
//
// Returns 0 on success.  -2 also covers a quota_per_chunk larger than chunk_rows * n (a chunk has
// no more entries than that; the count function above does not know n and cannot check it).  -7 means the request needs more than SB_NOALLOC_MAX_CHUNKS chunks and
// was rejected before anything was launched; other negative values are argument errors as in
// sb_residual_topk; positive values are CUDA error codes.
//
// The function calls no cudaMalloc, cudaFree or other allocating routine.  The first call on each
// device looks up the address of the built-in scratch array (once, with that device current);
// make that first call before starting any stream capture.  All calls on a device share the
// scratch array, which keeps the previous call's contents: the function clears what must start
// at zero itself, but two calls whose kernels overlap on the GPU (different streams without an
// ordering between them) race on it and must not be issued.
int sb_residual_topk_noalloc(const void* x, const void* c, const void* q, int rows, int n, int r, int ldx, int chunk_rows,
                             int quota_per_chunk, int bits, int* idx32, long long* idx64, void* val, float* scale, int* status,
                             void* stream);

#ifdef __cplusplus
}
#endif
