// Index checks of the debug build.
//
// The release kernels resolve a bad index quietly (an out-of-range token id is clamped, a page index
// beyond the cache reads the zero row, a target id outside the vocabulary gets log-prob of -inf) so that
// one bad element cannot fault the GPU. A library built with -DTX_DEBUG (`python -m tunix_b200.build_kernels
// --debug`, loaded with TUNIX_B200_DEBUG_KERNELS=1) additionally RECORDS the first such event of every
// translation unit: which check fired and the offending value. The host reads and clears the records through
// the exported `tx_debug_read_<unit>` functions (`ops._lib.check_status` does, and raises).
#pragma once

#include <cuda_runtime.h>

#ifdef TX_DEBUG
// One record per translation unit: {armed, check code, offending value, limit}.
#define TX_DEBUG_UNIT(unit)                                                                  \
  static __device__ int tx_dbg_record[4];                                                    \
  extern "C" int tx_debug_read_##unit(int* out4) {                                           \
    int h[4] = {0, 0, 0, 0};                                                                 \
    if (cudaMemcpyFromSymbol(h, tx_dbg_record, sizeof(h)) != cudaSuccess) return -1;         \
    const int z[4] = {0, 0, 0, 0};                                                           \
    if (h[0] && cudaMemcpyToSymbol(tx_dbg_record, z, sizeof(z)) != cudaSuccess) return -1;   \
    for (int i = 0; i < 4; ++i) out4[i] = h[i];                                              \
    return h[0];                                                                             \
  }
#define TX_DEBUG_CHECK(ok, code, value, limit)                                               \
  do {                                                                                       \
    if (!(ok) && atomicCAS(&tx_dbg_record[0], 0, 1) == 0) {                                  \
      tx_dbg_record[1] = (code);                                                             \
      tx_dbg_record[2] = static_cast<int>(value);                                            \
      tx_dbg_record[3] = static_cast<int>(limit);                                            \
    }                                                                                        \
  } while (0)
#else
#define TX_DEBUG_UNIT(unit)
#define TX_DEBUG_CHECK(ok, code, value, limit) do { } while (0)
#endif

// Check codes.
#define TX_DBG_TOKEN_ID 1      // embedding: token id outside [0, vocabulary)
#define TX_DBG_TARGET_ID 2     // log-prob: target id outside [0, vocabulary)
#define TX_DBG_PAGE_INDEX 3    // paged attention: block-table entry outside [0, pages)
#define TX_DBG_SLOT 4          // KV page write: slot beyond the cache
