/* Allocation-free routing plan for callers that must not allocate device memory.
 *
 * This entry point has no counterpart in the reference project; it exists for embedders of this
 * library that run inside someone else's memory budget: a serving process whose allocator owns all
 * of the device memory up front, a plugin called from a runtime that forbids cudaMalloc after
 * start-up, or code running on a stream where an allocation (which may synchronise the device)
 * is not acceptable.  Such callers cannot use the Python binding `moe_plan`, because that binding
 * allocates its outputs and a scratch buffer through the framework allocator on every call.
 *
 * What it computes is exactly what `moe_plan` computes: from the `[tokens, top_k]` expert choices
 * it derives the expert-sorted, 128-row padded row layout used by the grouped expert GEMMs
 *     row_token [capacity_rows]       source token of each sorted row, -1 for padding
 *     token_rows[tokens * top_k]      sorted row of each route
 *     tile_group[capacity_rows / 128] expert owning each 128-row tile
 *     group_rows[experts + 1]         first row of every expert segment
 *     meta      [>= 3]                live 128-row tiles, live rows, overflow flag
 * The caller owns and passes every input and output buffer (device pointers, int32).
 *
 * Scratch: the per-block expert histogram lives in one fixed array inside the library's device
 * image (256 KiB, reserved on every GPU that loads the library until the process exits).  The
 * limit that follows from its size:  tokens * top_k <= 1,048,576  and  experts <= 64.
 * Larger requests are refused (return value -1 and a message on stderr); nothing is launched.
 *
 * The first call made on a device looks up the device address of that array
 * (cudaGetSymbolAddress, with the caller's device current).  Make that first call outside any
 * stream capture.  No call allocates or frees memory.
 *
 * All calls on a device share the one scratch array.  It is fully rewritten by each call, so it
 * needs no clearing, but two calls whose kernels may overlap on the GPU (different streams, no
 * dependency between them) race on it: serialise them.
 *
 * Returns 0 on success, -1 size beyond the limit, -2 invalid argument, otherwise a cudaError_t.
 */
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

__attribute__((visibility("default"))) int mts_moe_plan_noalloc(
    const int* indices, int tokens, int top_k, int experts, int capacity_rows, int* row_token, int* token_rows,
    int* tile_group, int* group_rows, int* meta, void* cuda_stream);

#ifdef __cplusplus
}
#endif
