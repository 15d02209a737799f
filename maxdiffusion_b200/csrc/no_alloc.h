// Column sums for callers that cannot allocate device memory.
//
// This entry point has no counterpart in the reference (which has no native code at all). It exists for
// host programs that embed the kernel library in a context where cudaMalloc is off limits: code running
// inside a CUDA-graph capture or another framework's stream callback, plug-ins that must not disturb the
// host application's memory pool, and real-time loops that forbid allocation after start-up. The regular
// entry point `mdb_colsum` asks such callers for a scratch buffer sized by the launch geometry; this one
// keeps its scratch in a fixed array that lives inside the library image instead.
//
// What to know before using it:
//   * limit: at most MDB_COLSUM_NOALLOC_MAX_COLS columns (a multiple of 8); wider inputs are refused with
//     MDB_NOALLOC_ERR_TOO_WIDE and nothing is launched. The number of rows is not limited.
//   * cost: every GPU that loads the library holds the scratch array (2 MiB) until the process exits.
//   * the first call on a device looks up the device address of the scratch array (with that device
//     current). Make that first call outside of any stream capture.
//   * all calls on a device share the one array. The kernel rewrites every partial sum it later reads, so
//     nothing needs clearing between calls, but two calls that overlap on the GPU (different streams, or a
//     graph replayed concurrently) race on the array; serialise them.
//   * it calls no cudaMalloc / cudaFree and no allocating library routine; inputs and outputs are the
//     caller's: x is bf16 [rows, cols] with leading dimension ldx (elements), out is fp32 [cols].
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define MDB_COLSUM_NOALLOC_MAX_COLS 8192
#define MDB_COLSUM_NOALLOC_CTAS 64

#define MDB_NOALLOC_OK 0
#define MDB_NOALLOC_ERR_TOO_WIDE (-1)      /* cols > MDB_COLSUM_NOALLOC_MAX_COLS */
#define MDB_NOALLOC_ERR_BAD_SHAPE (-2)     /* cols <= 0, cols not a multiple of 8, or ldx < cols */
#define MDB_NOALLOC_ERR_SETUP (-3)         /* the scratch array's device address could not be obtained */

/* Returns MDB_NOALLOC_OK, one of the negative codes above, or a positive cudaError_t from the launch. */
int mdb_colsum_noalloc(const void* x, long long ldx, int rows, int cols, float* out, void* stream);

/* Human-readable text for a return value of mdb_colsum_noalloc. */
const char* mdb_colsum_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
