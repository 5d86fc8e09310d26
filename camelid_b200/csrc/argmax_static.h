/* Greedy token choice for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in karan68/Camelid: it exists for users of this
 * library whose code runs where cudaMalloc is off limits. Examples are a plug-in that lives
 * inside another program's CUDA context and is handed a fixed memory budget, a real-time
 * loop that may not call into the allocator (its latency is unbounded and it can
 * synchronise the device), and a host that has already given all device memory to a pool of
 * its own. Such a caller owns the logits and the output buffer and passes them in; the
 * only other memory the kernel needs, two 64-bit words per row in which the blocks of a
 * row meet, lives in a fixed array inside the library (16 bytes x
 * CML_ARGMAX_STATIC_MAX_ROWS = 64 KiB per GPU, held from the moment the library is loaded
 * on that GPU until the process ends).
 *
 *   logits  device pointer, float32 [rows, ld] (ld >= vocab), row-major
 *   out     device pointer, int32 [rows]: index of the largest logit of each row, the lowest
 *           index among equal maxima
 *   err     device pointer, int32 [1]: bit 0 is set if a logit is not finite (may not be null)
 *   stream  cudaStream_t of the current device
 *   msg     optional host buffer for a message when the call is refused (may be null)
 *
 * Returns 0, a cudaError_t (> 0), or CML_ARGMAX_STATIC_TOO_MANY_ROWS / _BAD_ARGUMENT.
 *
 * Rules that follow from the fixed array:
 *  - rows above CML_ARGMAX_STATIC_MAX_ROWS are refused; nothing is launched.
 *  - All calls on one GPU share the array. Calls whose kernels can run at the same time
 *    (different streams, no event between them) race on it and give wrong tokens; calls on
 *    one stream, or ordered by events, are fine.
 *  - The array keeps what the last call left. A completed call leaves it zero, but a call
 *    that was cut short may not, so every call first clears the words it is going to use
 *    (a memset node on the same stream).
 *  - The first call on each GPU looks up the array's device address
 *    (cudaGetSymbolAddress, with that GPU current). Make that first call outside any
 *    stream capture; later calls only enqueue a memset and a kernel.
 *  - The address is remembered per GPU ordinal and belongs to the context the CUDA runtime
 *    uses on that GPU (its primary context). A caller that creates further driver-API
 *    contexts on the same GPU must call this only with the primary context current; from
 *    another context the remembered address is not valid.
 *  - The call allocates nothing: no cudaMalloc, cudaFree or library routine that allocates.
 *  - Every refusal and every failed CUDA call leaves a message in msg (when msg is given).
 */
#ifndef CAMELID_B200_ARGMAX_STATIC_H
#define CAMELID_B200_ARGMAX_STATIC_H

#define CML_ARGMAX_STATIC_MAX_ROWS 4096
#define CML_ARGMAX_STATIC_TOO_MANY_ROWS (-10)
#define CML_ARGMAX_STATIC_BAD_ARGUMENT (-11)

#ifdef __cplusplus
extern "C" {
#endif

int cml_argmax_rows_static(const float* logits, int ld, int rows, int vocab, int* out, int* err, void* stream,
                           char* msg, int msg_len);

#ifdef __cplusplus
}
#endif
#endif
