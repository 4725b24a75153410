/* C declarations of entry points of libninfer_b200.so that are meant to be called from
 * outside the Python package.  Every function returns 0 on success; on failure it returns
 * non-zero and nf_last_error() gives the reason as text. */
#pragma once

#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* nf_last_error(void);

/* Decode attention (one query row per request, bfloat16, paged cache) with caller-provided
 * scratch: ws_acc float32 [T, Hq, nsplit, D], ws_ml float32 [T, Hq, nsplit, 2].
 *
 * nsplit is the number of blocks of 128 keys the scratch has room for per row and head; it
 * must be at least ceil((largest position + 1) / 128) over the rows of the call.  Positions
 * live on the device, so the host cannot check this: a row that needs more blocks is
 * computed over its first nsplit * 128 keys only, nothing is written outside the scratch,
 * and nf_decode_attention_status() reports 1 + that row afterwards.
 *
 * Inside a stream capture the library chains its kernels (each may begin while the one before it
 * drains) and these kernels read `positions` and the row list before they wait for their
 * predecessor: those two must have been written before the kernel that precedes this call in the
 * stream was launched (by a copy at the start of the step, as the engine does), not by it. */
int nf_decode_attention(const void* qkv, int q_row_stride, const void* pages, const int* block_table,
                        int bt_width, const int* positions, const int* row_seg, void* out,
                        float* ws_acc, float* ws_ml, int T, int Hq, int Hkv, int D, int page_size,
                        int num_pages, int window, float scale, int nsplit, cudaStream_t stream);

/* The same computation for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference engine.
 *
 * Who needs it: code that runs where cudaMalloc is off limits - a plug-in inside a host
 * application that has handed the whole device budget to its own pool, a control loop that
 * cannot tolerate the device-wide synchronisation and jitter an allocation may bring, or a
 * process whose sandbox denies further device allocations after start-up.  Such callers
 * still pass their own inputs and the output buffer; only the kernel's scratch (partial
 * results per block of 128 keys) is taken care of: it lives in a fixed array inside the
 * library, nf_decode_attention_static_scratch_bytes() bytes that every GPU which loads the
 * library holds until the process exits.
 *
 * Limits and rules:
 *   - T * Hq * nsplit * (D + 2) * 4 bytes must fit the fixed array; larger calls are
 *     refused with an error, nothing is launched.
 *   - nsplit follows the rule given at nf_decode_attention: at least
 *     ceil((largest position + 1) / 128) over the rows of the call.
 *   - The first call on each device looks up the array's device address.  Make that first
 *     call with the device current and before any stream capture begins.
 *   - No cudaMalloc, cudaFree or allocating library routine is called, on any call.
 *   - All calls share the one array.  The kernels overwrite every element they later read,
 *     so nothing has to be cleared between calls; but two calls whose kernels overlap on the
 *     GPU (different streams, no ordering between them) race on it.  Order them. */
int nf_decode_attention_static(const void* qkv, int q_row_stride, const void* pages,
                               const int* block_table, int bt_width, const int* positions,
                               const int* row_seg, void* out, int T, int Hq, int Hkv, int D,
                               int page_size, int num_pages, int window, float scale, int nsplit,
                               cudaStream_t stream);

/* 0, or 1 + the first row whose position needed more key blocks than a call's nsplit gave,
 * since the last call of this function.  Reads and clears; synchronises the device. */
int nf_decode_attention_status(void);

/* Size of the fixed scratch array in bytes. */
long long nf_decode_attention_static_scratch_bytes(void);

#ifdef __cplusplus
}
#endif
