/* An entry point of the kernel library that allocates no memory.
 *
 * It has no counterpart in the reference (lateos-ai/reflex allocates its
 * attention partials per call through its CUDA bindings); it is this library's
 * own addition.
 *
 * Who it is for.  Every other entry point of this library leaves allocation to
 * its caller, and the Python layer allocates through torch's caching
 * allocator.  Some callers cannot do that:
 *   - a host program that hands the whole device to an arena of its own when
 *     it starts, so that a later cudaMalloc fails;
 *   - a latency-critical loop in which cudaMalloc and cudaFree are not
 *     acceptable because they may synchronise the device;
 *   - a plain C caller that links the library without torch and has no
 *     allocator to lend.
 * For them the split-KV decode attention, whose splits exchange partial
 * results through scratch memory, is offered with that scratch built into the
 * library.
 *
 * The scratch is one file-scope device array of RFX_NOALLOC_SCRATCH_FLOATS
 * floats (4 MiB).  Every GPU on which the library is loaded holds it until the
 * process exits.  A call needs  R * nq * n_splits * (head_dim + 2)  floats when
 * n_splits > 1 and nothing otherwise; a call that needs more is refused with
 * RFX_ERR_SCRATCH (-4) and launches nothing.
 *
 * First call on a device.  The first call made with a given device current
 * looks up the array's device address (cudaGetSymbolAddress) and keeps it; do
 * that first call outside of any stream capture.  Later calls only launch.
 *
 * Sharing.  All calls on a device use the same array, and it keeps whatever
 * the last call left.  Nothing in it has to be zero: each call overwrites all
 * that it reads.  Two calls that may run on the GPU at the same time (different
 * streams, or different host threads without ordering between their streams)
 * race on the array; order them on one stream or with events.
 *
 * The entry point calls no cudaMalloc, cudaFree or other allocating routine.
 * Inputs and outputs are the caller's, as in rfx_attention_decode:
 *   q, out      bfloat16 [R, nq, head_dim]
 *   k_pages,    bfloat16 [pages, nkv, 64, head_dim]
 *   v_pages
 *   page_table  int32 [slots, max_pages]; row_pos, row_slot int32 [R]
 * Returns 0, a cudaError_t, or a negative library code (see
 * rfx_error_string).
 */
#ifndef REFLEX_B200_NOALLOC_H
#define REFLEX_B200_NOALLOC_H

#define RFX_NOALLOC_SCRATCH_FLOATS (1u << 20)

#ifdef __cplusplus
extern "C" {
#endif

int rfx_attention_decode_noalloc(const void* q, const void* k_pages, const void* v_pages,
                                 const int* page_table, int max_pages, int page_size,
                                 const int* row_pos, const int* row_slot, void* out, int R, int nq,
                                 int nkv, int head_dim, int n_splits, int window, float scale,
                                 void* stream);

/* The array's size in floats (RFX_NOALLOC_SCRATCH_FLOATS), for callers that
 * size their splits against it. */
long long rfx_attention_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif

#endif
