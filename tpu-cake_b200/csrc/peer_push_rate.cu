// peer_push_rate: how fast can every GPU of a node push to every other GPU at once, in the access
// pattern of the matmul epilogue? The answer is the link-side denominator of the fused matmul +
// reduce-scatter step and it decided two things in cake_matmul_rs_sm100: that the arrival flags are
// released by a publisher warp and not by the pushing threads, and that tensor stores of 32 rows x
// 128 bytes are kept.
//
// One process drives all GPUs (peer access, no NCCL). Every GPU runs 148 blocks x 4 pushing warps;
// warp w sends chunk after chunk (32 rows of a [2048, 16 KiB] destination per peer and source)
// round-robin to its peers, 32 MiB to each. Nothing waits on another GPU: a launch ends when its
// own stores have completed. Times are CUDA events around each GPU's launch; the slowest GPU counts.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -o peer_push_rate peer_push_rate.cu
//   ./peer_push_rate [GPUs]
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include <vector>

#define CHECK(call)                                                              \
  do {                                                                           \
    cudaError_t status_ = (call);                                                \
    if (status_ != cudaSuccess) {                                                \
      printf("%s failed: %s\n", #call, cudaGetErrorString(status_));             \
      exit(1);                                                                   \
    }                                                                            \
  } while (0)

namespace {

constexpr int kBlocks = 148;
constexpr int kPushWarps = 4;
constexpr int kRows = 2048;          // rows of one destination
constexpr int kPitch = 16384;        // bytes per row
constexpr int kMaxPeers = 7;

struct alignas(64) PeerMaps {
  CUtensorMap map[kMaxPeers];
};

struct PeerPointers {
  char* data[kMaxPeers];
  uint32_t* flags[kMaxPeers];
};

enum Store { kPlain = 0, kTensor2d = 1, kTensor3d = 2 };
enum Announce {
  kNone = 0,          // nothing
  kWaitFence = 1,     // every 4 chunks: wait for the 4 before, proxy fence (tensor stores only)
  kRelaxedFlag = 2,   // kWaitFence + st.relaxed.sys of a flag at the peer
  kReleaseFlag = 3,   // kWaitFence + st.release.sys of a flag at the peer
  kFenceWarp = 4,     // kWaitFence, and a fifth warp that fences at system scope and writes a relaxed flag every microsecond
};

struct Variant {
  int store;
  int announce;
  int row_bytes;  // bytes one chunk covers per row: 128, 256 or 512
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__global__ void __launch_bounds__((kPushWarps + 1) * 32)
push_kernel(const __grid_constant__ PeerMaps maps, PeerPointers peers_of, int peers, Variant v, int chunks_per_peer) {
  extern __shared__ uint8_t raw[];
  __shared__ int finished;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) finished = 0;
  __syncthreads();
  if (warp == kPushWarps) {
    if (v.announce != kFenceWarp || lane != 0) return;
    uint32_t n = 0;
    while (atomicAdd(&finished, 0) < kPushWarps) {
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(peers_of.flags[n % peers] + 1000 + (blockIdx.x & 15)), "r"(n) : "memory");
      ++n;
      __nanosleep(1000);
    }
    return;
  }
  const int chunk_bytes = 32 * v.row_bytes;
  uint8_t* staging = base + warp * 2 * chunk_bytes;
  for (int i = lane; i < 2 * chunk_bytes / 4; i += 32) reinterpret_cast<uint32_t*>(staging)[i] = i;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  const int warps = gridDim.x * kPushWarps;
  const int w = blockIdx.x * kPushWarps + warp;
  const int chunks_per_row = kPitch / v.row_bytes;
  const int per_warp = (chunks_per_peer + warps - 1) / warps;
  const uint4 value = make_uint4(1, 2, 3, 4);
  int count = 0;
  bool pending = false;
  for (int k = 0; k < per_warp * peers; ++k) {
    const int peer = k % peers;
    const long long c = static_cast<long long>(k / peers) * warps + w;
    if (c >= chunks_per_peer) continue;
    const int row_block = static_cast<int>(c / chunks_per_row), piece = static_cast<int>(c % chunks_per_row);
    if (v.store == kPlain) {
      char* dst = peers_of.data[peer] + static_cast<size_t>(row_block) * 32 * kPitch + piece * 128;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = i * 4 + lane / 8;
        *reinterpret_cast<uint4*>(dst + static_cast<size_t>(r) * kPitch + (lane % 8) * 16) = value;
      }
    } else if (lane == 0) {
      if (count >= 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      const uint32_t src = smem_u32(staging + (count & 1) * chunk_bytes);
      const uint64_t map = reinterpret_cast<uint64_t>(&maps.map[peer]);
      if (v.store == kTensor3d) {
        asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                     ::"l"(map), "r"(src), "r"(0), "r"(piece * (v.row_bytes / 128)), "r"(row_block * 32) : "memory");
      } else {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                     ::"l"(map), "r"(src), "r"(piece * (v.row_bytes / 2)), "r"(row_block * 32) : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    ++count;
    if ((count & 3) == 0 && lane == 0 && v.announce != kNone) {
      uint32_t* flag = peers_of.flags[peer] + (w & 511);
      if (v.store == kPlain) {
        if (v.announce == kReleaseFlag) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(count) : "memory");
        if (v.announce == kRelaxedFlag) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(count) : "memory");
      } else {
        if (pending) {
          asm volatile("cp.async.bulk.wait_group 4;" ::: "memory");
          asm volatile("fence.proxy.async.global;" ::: "memory");
          if (v.announce == kReleaseFlag) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(count) : "memory");
          if (v.announce == kRelaxedFlag) asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(count) : "memory");
        }
        pending = true;
      }
    }
  }
  if (v.store != kPlain && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  __syncwarp();
  if (lane == 0) atomicAdd(&finished, 1);
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

bool encode_map(EncodeTiled encode, CUtensorMap* map, char* base, const Variant& v) {
  const cuuint32_t ones[3] = {1, 1, 1};
  if (v.store == kTensor3d) {
    // (64 bf16, 128-byte pieces of a row, rows): one box is 32 rows x row_bytes, written piece by piece
    const cuuint64_t dims[3] = {64, kPitch / 128, kRows};
    const cuuint64_t strides[2] = {128, kPitch};
    const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(v.row_bytes / 128), 32};
    return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
  }
  const cuuint64_t dims[2] = {kPitch / 2, kRows};
  const cuuint64_t strides[1] = {kPitch};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(v.row_bytes / 2), 32};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
                v.row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

int main(int argc, char** argv) {
  int present = 0;
  CHECK(cudaGetDeviceCount(&present));
  const int world = argc > 1 ? atoi(argv[1]) : present;
  if (world < 2 || world > present || world > kMaxPeers + 1) {
    printf("needs 2..%d GPUs, asked for %d of %d\n", kMaxPeers + 1, world, present);
    return 1;
  }
  const int peers = world - 1;
  const size_t per_peer = static_cast<size_t>(kRows) * kPitch;
  void* symbol = nullptr;
  cudaDriverEntryPointQueryResult found;
  CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &symbol, cudaEnableDefault, &found));
  if (symbol == nullptr) {
    printf("cuTensorMapEncodeTiled is not available\n");
    return 1;
  }
  const EncodeTiled encode = reinterpret_cast<EncodeTiled>(symbol);

  std::vector<char*> receive(world);
  std::vector<uint32_t*> flags(world);
  std::vector<cudaStream_t> stream(world);
  std::vector<cudaEvent_t> begin(world), end(world);
  for (int r = 0; r < world; ++r) {
    CHECK(cudaSetDevice(r));
    for (int p = 0; p < world; ++p) {
      if (p == r) continue;
      const cudaError_t enabled = cudaDeviceEnablePeerAccess(p, 0);
      if (enabled != cudaSuccess && enabled != cudaErrorPeerAccessAlreadyEnabled) {
        printf("GPU %d cannot reach GPU %d: %s\n", r, p, cudaGetErrorString(enabled));
        return 1;
      }
      cudaGetLastError();
    }
    CHECK(cudaMalloc(&receive[r], per_peer * world));
    CHECK(cudaMalloc(&flags[r], 8192 * world));
    CHECK(cudaMemset(flags[r], 0, 8192 * world));
    CHECK(cudaStreamCreate(&stream[r]));
    CHECK(cudaEventCreate(&begin[r]));
    CHECK(cudaEventCreate(&end[r]));
    CHECK(cudaFuncSetAttribute(push_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
  }

  struct Case {
    Variant v;
    const char* name;
  };
  const Case cases[] = {
      {{kPlain, kNone, 128}, "16-byte stores"},
      {{kPlain, kReleaseFlag, 128}, "16-byte stores, st.release.sys flag per 4 chunks"},
      {{kTensor2d, kNone, 128}, "tensor stores 32 x 128 B"},
      {{kTensor2d, kWaitFence, 128}, "tensor stores, wait + proxy fence per 4 chunks"},
      {{kTensor2d, kReleaseFlag, 128}, "tensor stores, wait + fence + st.release.sys flag"},
      {{kTensor2d, kRelaxedFlag, 128}, "tensor stores, wait + fence + st.relaxed.sys flag"},
      {{kTensor2d, kFenceWarp, 128}, "tensor stores, wait + fence; a fifth warp releases"},
      {{kTensor3d, kNone, 256}, "tensor stores 32 x 2 x 128 B (3-D map)"},
      {{kTensor3d, kNone, 512}, "tensor stores 32 x 4 x 128 B (3-D map)"},
      {{kTensor2d, kNone, 256}, "tensor stores 32 x 256 B, unswizzled"},
      {{kTensor2d, kNone, 512}, "tensor stores 32 x 512 B, unswizzled"},
      {{kTensor2d, kNone, 128}, "tensor stores 32 x 128 B (again)"},
  };
  for (const Case& c : cases) {
    std::vector<PeerMaps> maps(world);
    std::vector<PeerPointers> pointers(world);
    for (int r = 0; r < world; ++r) {
      for (int k = 0; k < peers; ++k) {
        const int destination = (r + 1 + k) % world;
        pointers[r].data[k] = receive[destination] + static_cast<size_t>(r) * per_peer;
        pointers[r].flags[k] = flags[destination] + static_cast<size_t>(r) * 2048;
        if (c.v.store != kPlain && !encode_map(encode, &maps[r].map[k], pointers[r].data[k], c.v)) {
          printf("tensor map refused for %s\n", c.name);
          return 1;
        }
      }
    }
    const int chunks_per_peer = static_cast<int>(per_peer / (32 * c.v.row_bytes));
    const size_t smem = static_cast<size_t>(kPushWarps) * 2 * 32 * c.v.row_bytes + 1024;
    for (int repeat = 0; repeat < 3; ++repeat) {
      for (int r = 0; r < world; ++r) {
        CHECK(cudaSetDevice(r));
        CHECK(cudaEventRecord(begin[r], stream[r]));
        push_kernel<<<kBlocks, (kPushWarps + 1) * 32, smem, stream[r]>>>(maps[r], pointers[r], peers, c.v, chunks_per_peer);
        CHECK(cudaEventRecord(end[r], stream[r]));
      }
      for (int r = 0; r < world; ++r) {
        CHECK(cudaSetDevice(r));
        CHECK(cudaStreamSynchronize(stream[r]));
        CHECK(cudaGetLastError());
      }
    }
    float slowest = 0.f, fastest = 1e9f;
    for (int r = 0; r < world; ++r) {
      float ms = 0.f;
      CHECK(cudaEventElapsedTime(&ms, begin[r], end[r]));
      slowest = ms > slowest ? ms : slowest;
      fastest = ms < fastest ? ms : fastest;
    }
    const double bytes = static_cast<double>(per_peer) * peers;
    printf("%d GPUs | %-52s | %.0f MB out per GPU | slowest GPU %.3f ms = %.0f GB/s, fastest %.0f GB/s\n", world, c.name,
           bytes / 1e6, slowest, bytes / slowest / 1e6, bytes / fastest / 1e6);
    fflush(stdout);
  }
  return 0;
}
