// Host-side helpers shared by the translation units of libcake_b200.so: thread-local error
// text, CUDA error mapping, and access to the driver's tensor-map encoder without linking
// libcuda directly.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>

#include "../../include/cake_abi.h"

namespace cake {

// Stores a printf-formatted message as the calling thread's last error and returns `code`.
int32_t fail(int32_t code, const char* fmt, ...);

#define CAKE_CUDA_TRY(expr)                                                                  \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess) {                                                                 \
      return ::cake::fail(CAKE_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                          __FILE__, __LINE__);                                               \
    }                                                                                        \
  } while (0)

// Encodes a tiled tensor map (bf16 elements unless elem_bytes says otherwise) through the
// driver entry point resolved at run time. dims/strides are innermost-first; strides are in
// bytes and omit the innermost dimension.
int32_t encode_tensor_map(CUtensorMap* out, const void* base, uint32_t rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128);

// Same, with the element size given: 2 = bfloat16, 4 = float32.
int32_t encode_tensor_map_typed(CUtensorMap* out, const void* base, uint32_t rank, const uint64_t* dims,
                                const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128,
                                int elem_bytes);

// Device status word helpers (4 x int32 in device memory).
struct StatusWord {
  int32_t* dev = nullptr;
  int32_t ensure();
  int32_t read_and_clear(cudaStream_t stream, cake_status* out);
  void release();
};

}  // namespace cake
