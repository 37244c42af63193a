// General entry points of libcake_b200.so: error text, symmetric allocations and their CUDA IPC
// export/import, the tensor-map encoder and the device status word.
#include <stdio.h>
#include <string.h>

#include "cake_host.h"

namespace cake {

static thread_local char g_last_error[512] = "";

int32_t fail(int32_t code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
  va_end(ap);
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn resolve_encoder() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult q;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || sym == nullptr) return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(sym);
  return fn;
}

int32_t encode_tensor_map(CUtensorMap* out, const void* base, uint32_t rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128) {
  return encode_tensor_map_typed(out, base, rank, dims, strides_bytes, box, swizzle128, 2);
}

int32_t encode_tensor_map_typed(CUtensorMap* out, const void* base, uint32_t rank, const uint64_t* dims,
                                const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128,
                                int elem_bytes) {
  EncodeTiledFn fn = resolve_encoder();
  if (!fn) return fail(CAKE_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (uint32_t i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) gstrides[i] = strides_bytes[i];
  }
  CUresult r = fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, rank, const_cast<void*>(base), gdims,
                  gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    return fail(CAKE_ERR_CUDA,
                "cuTensorMapEncodeTiled failed with CUresult %d (rank %u, dims %llu x %llu, box %u x %u)",
                static_cast<int>(r), rank, static_cast<unsigned long long>(dims[0]),
                static_cast<unsigned long long>(rank > 1 ? dims[1] : 1), box[0], rank > 1 ? box[1] : 1);
  }
  return CAKE_OK;
}

int32_t StatusWord::ensure() {
  if (dev) return CAKE_OK;
  CAKE_CUDA_TRY(cudaMalloc(&dev, 4 * sizeof(int32_t)));
  CAKE_CUDA_TRY(cudaMemset(dev, 0, 4 * sizeof(int32_t)));
  return CAKE_OK;
}

int32_t StatusWord::read_and_clear(cudaStream_t stream, cake_status* out) {
  int32_t host[4] = {0, 0, 0, 0};
  if (dev) {
    CAKE_CUDA_TRY(cudaMemcpyAsync(host, dev, sizeof(host), cudaMemcpyDeviceToHost, stream));
    CAKE_CUDA_TRY(cudaMemsetAsync(dev, 0, sizeof(host), stream));
    CAKE_CUDA_TRY(cudaStreamSynchronize(stream));
  }
  out->code = host[0];
  out->detail0 = host[1];
  out->detail1 = host[2];
  out->detail2 = host[3];
  return CAKE_OK;
}

void StatusWord::release() {
  if (dev) cudaFree(dev);
  dev = nullptr;
}

}  // namespace cake

extern "C" {

int32_t cake_abi_version(void) { return 1; }

const char* cake_last_error(void) { return cake::g_last_error; }

int32_t cake_symm_alloc(size_t bytes, void** out_ptr) {
  if (!out_ptr || bytes == 0) return cake::fail(CAKE_ERR_INVALID_ARGUMENT, "cake_symm_alloc: bad arguments");
  void* p = nullptr;
  CAKE_CUDA_TRY(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cake::fail(CAKE_ERR_CUDA, "cudaMemset failed: %s", cudaGetErrorString(e));
  }
  CAKE_CUDA_TRY(cudaDeviceSynchronize());
  *out_ptr = p;
  return CAKE_OK;
}

int32_t cake_symm_free(void* ptr) {
  if (ptr) CAKE_CUDA_TRY(cudaFree(ptr));
  return CAKE_OK;
}

int32_t cake_ipc_export(void* ptr, uint8_t handle_out[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  if (!ptr || !handle_out) return cake::fail(CAKE_ERR_INVALID_ARGUMENT, "cake_ipc_export: null argument");
  cudaIpcMemHandle_t h;
  CAKE_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle_out, &h, 64);
  return CAKE_OK;
}

int32_t cake_ipc_open(const uint8_t handle[64], void** out_ptr) {
  if (!handle || !out_ptr) return cake::fail(CAKE_ERR_INVALID_ARGUMENT, "cake_ipc_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  CAKE_CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out_ptr = p;
  return CAKE_OK;
}

int32_t cake_ipc_close(void* ptr) {
  if (ptr) CAKE_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return CAKE_OK;
}

}  // extern "C"
