// se_moe_route_build_no_alloc: the routing build of the expert layers for callers that
// cannot allocate device memory.
//
// This entry point has no counterpart in CURRENTF/SparseEngine; it is an addition of this
// library.
//
// Who it is for.  The ordinary entry point, se_moe_route_build, takes two scratch arrays
// from its caller (per-expert counts and per-assignment ranks), and the Python bindings
// get them from the framework's allocator.  Some callers have no allocator to ask at the
// moment of the call: code that runs where cudaMalloc is forbidden or would synchronise
// the device (inside a latency-critical loop, in a host callback, in a process that was
// handed a fixed memory budget and spent it), plain C programs that link this library
// without any tensor framework, and code that must not disturb the memory pools of the
// process it is embedded in.  For them the scratch lives inside the library: a file-scope
// device array of fixed size.  The caller still passes its input and every output.
//
// What it costs and what it limits.
//   * The array holds SE_NOALLOC_MAX_EXPERTS + SE_NOALLOC_MAX_ASSIGNMENTS ints (about
//     260 KB).  Every GPU on which the library is loaded keeps it until the process exits.
//   * Larger problems are refused with an error code (below); use se_moe_route_build then.
//   * The entry point calls no cudaMalloc, no cudaFree and no allocating library routine.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current).  Make that first call outside any
//     stream capture, and from one thread per device.
//   * All calls share the one array, which keeps whatever the last call left in it.  The
//     kernels overwrite all of it that they later read, so nothing needs clearing, but two
//     calls whose kernels overlap on the GPU (different streams, or threads racing on one
//     device) would race on it: issue the calls of one device on one stream, or order them.
//   * ids must lie in [0, experts), as for se_moe_route_build.
//
// Arguments (all device pointers, int32): ids[assignments] is the expert of assignment
// a = token * top_k + slot; outputs offsets[experts + 1], sorted[assignments],
// inv_pos[assignments], tile_expert[max_tiles], tile_row0[max_tiles], num_tiles[1] with
// max_tiles = ceil(assignments / tile_rows) + min(experts, assignments) — the same
// outputs, bit for bit, as se_moe_route_build.  Returns 0, a positive cudaError_t, or one
// of the negative codes below; se_no_alloc_strerror turns any of them into text.
#pragma once
#include <cuda_runtime.h>

#define SE_NOALLOC_MAX_EXPERTS 1024
#define SE_NOALLOC_MAX_ASSIGNMENTS 65536

#define SE_NOALLOC_ERR_ARGUMENT (-10)
#define SE_NOALLOC_ERR_TOO_MANY_ASSIGNMENTS (-11)
#define SE_NOALLOC_ERR_TOO_MANY_EXPERTS (-12)
#define SE_NOALLOC_ERR_DEVICE (-13)

#ifdef __cplusplus
extern "C" {
#endif
int se_moe_route_build_no_alloc(const int* ids, int assignments, int experts, int tile_rows, int* offsets, int* sorted,
                                int* inv_pos, int* tile_expert, int* tile_row0, int* num_tiles, cudaStream_t stream);
const char* se_no_alloc_strerror(int code);
#ifdef __cplusplus
}
#endif
