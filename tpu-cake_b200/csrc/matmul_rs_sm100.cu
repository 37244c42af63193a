// K-sharded BF16 matmul followed by a reduce-scatter, for sm_100a.
//
// What it replaces: the local contraction `_matmul_kernel` (src/tpu_cake/pallas_lowering.py:44-50,
// launched :429-444) and the collective that follows it (lax.psum_scatter :459-464, or the
// bidirectional Pallas ring :117-326). The reference materialises the f32 partial [M,N] in HBM
// between the two; here the epilogue of the contraction writes every partial tile straight to the
// GPU that owns it, and six more warps of the same kernel sum the W received copies in rank order
// while the contraction is still running.
//
// cake_matmul_rs_sm100<BN, B_KMAJOR>: persistent, warp-specialised.
//   warp 0    TMA producer: A tile 128x64 and B tile 64xBN (bf16) per stage into 128B-swizzled smem
//   warp 1    owns TMEM; one lane issues tcgen05.mma (M=128, N=BN, K=16), f32 accumulators in TMEM,
//             two accumulator buffers so the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2-5 epilogue: tcgen05.ld -> convert -> swizzled smem staging -> 128-byte row segments to
//             the owner's receive slot (local or peer memory)
//   warps 6-11 slot reduction (peer-to-peer strategy): walk this rank's receive slots in the order
//             the peers fill them, out = sum over source ranks in fixed order (deterministic)
//
// Arrival is announced by flags, one 32-bit word per source rank and per quarter tile (32 rows x BN
// columns: what one epilogue warp sends of a tile), holding the number of the call whose data is in
// the slot. An epilogue warp publishes a quarter one tile late: by then the tensor stores that
// carried it have completed, so the warp never waits for the link, and the release store costs a
// fence but no drain. Flags only grow, slots alternate between two parities, and nothing is
// consumed destructively: a reduction that gave up can simply be enqueued again.
// cake_reduce_slots_sm100 is the same reduction as a kernel of its own, for hosts that enqueue
// the pushes of several mesh positions on one GPU before any reduction.
#include <cuda_bf16.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "cake_host.h"
#include "cake_ptx.cuh"

namespace cake {

constexpr int kTileM = 128;
constexpr int kBlockK = 64;  // 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;
// Producer, issuer, 4 epilogue warps, 6 reduction warps (the last of them first publishes the
// arrival flags, for as long as the epilogue warps run). Twelve warps are three per scheduler, whose
// register file (16 K) then allows 168 registers per thread -- the same as ten warps would get.
constexpr int kGemmThreads = 384;
constexpr uint32_t kABytes = kTileM * kBlockK * 2;
// Chunks (32 rows x 128 bytes) an epilogue warp can have staged for stores still reading shared
// memory, and the depth of the 256-wide configuration's operand ring: the two compete for the
// CTA's shared memory (4 stages + 2 chunks, or 3 stages + up to 5 chunks, fit; 3 + 4 measured
// 9 % slower in the contraction and no faster in the pushes).
#ifndef CAKE_MM_STAGING_CHUNKS
#define CAKE_MM_STAGING_CHUNKS 2
#endif
#ifndef CAKE_MM_STAGES_256
#define CAKE_MM_STAGES_256 4
#endif
constexpr int kStagingChunks = CAKE_MM_STAGING_CHUNKS;
constexpr uint32_t kStagingBytesPerWarp = kStagingChunks * 32 * 128;
constexpr long long kBarrierBudgetCycles = 4000000000ll;  // about two seconds of SM clock
constexpr unsigned long long kDefaultPeerBudgetMs = 20000ull;  // 20 s unless the descriptor says otherwise

template <int BN>
struct GemmCfg {
  static constexpr uint32_t kBBytes = BN * kBlockK * 2;
  static constexpr uint32_t kStageBytes = kABytes + kBBytes;
  static constexpr int kStages = BN == 256 ? CAKE_MM_STAGES_256 : (BN == 128 ? 6 : 8);
  static constexpr uint32_t kTmemCols = 2 * BN;  // 128, 256 or 512: a power of two >= 32
  static constexpr uint32_t kSmemBytes =
      kStages * kStageBytes + 4 * kStagingBytesPerWarp + 512 /*barriers, mailbox*/ + 1024 /*alignment*/;
};

// What the slot reduction needs: this rank's receive slots of the current parity (source s at
// slots + s * slot_stride, each a [out_rows, out_cols] array in the transport dtype), its arrival
// flags ([W sources][quarters], quarter ((mi * n_tiles + ni) * 4 + q) of the region's tile grid) and
// the output.
struct ReduceParams {
  const char* slots;
  void* out;
  const uint32_t* flags;
  unsigned long long slot_stride;  // bytes, a multiple of 128
  unsigned long long budget_ns;    // how long a quarter may stay unannounced before the reduction gives up
  uint32_t epoch;                  // the call number a flag must have reached
  int32_t quarters;                // flags per source
  int32_t out_rows, out_cols, world;
  int32_t in_f32, out_f32;  // transport / output element type: 1 = f32, 0 = bf16
  int32_t vec_ok;           // rows are whole 16-byte pieces, in groups of 8 rows, mesh of 2, 4 or 8
  int32_t tile_n;           // the pushing side's tile width (sets the order the slots fill in)
  int32_t* tickets;         // [0] next chunk to hand out, [1] blocks that have finished; both 0 between launches
  int32_t* status;
};

// MatmulParams::publish: 0 = destinations are not receive slots, nothing to announce.
constexpr int kPublishPerTile = 1;  // every epilogue warp announces its quarter, one tile late
// Announcements an epilogue warp may have handed to the publisher warp without their having been
// sent yet, and the bit of the hand-over counter that says the epilogue warp has finished.
constexpr uint32_t kMailDepth = 4;
constexpr uint32_t kMailDone = 0x80000000u;
constexpr int kPublisherWarp = 11;
constexpr int kPublishAtEnd = 2;    // the last block to finish announces everything (tiles may straddle owners)

struct MatmulParams {
  int32_t m, n, k_local;
  int32_t m_tiles, n_tiles, k_blocks;
  int32_t world, rank, scatter_dim;
  int32_t out_rows, out_cols;  // shape of one owner's local output
  int32_t store_f32;           // destination element type: 1 = f32, 0 = bf16
  int32_t vec_ok;              // 16-byte pieces never straddle owners or bounds
  int32_t tma_store;           // epilogue chunks leave shared memory as TMA tensor stores
  int32_t region_order;        // consecutive tiles go to consecutive owners, starting at rank+1
  int32_t owner_rotation;      // tile groups after which the owner sequence shifts by one
  int32_t own_tail;            // this many of the rank's own tiles (the last of its region) come after everything else
  int32_t region_tiles;        // tiles of one owner's region
  int32_t publish;             // kPublish*
  int32_t mailbox;             // kPublishPerTile: the release stores are issued by the publisher warp
  int32_t own_now;             // kPublishPerTile: quarters of the rank's own region are announced without the one-tile delay
  int32_t reduce_in_kernel;    // the slot reduction runs in this kernel
  uint32_t epoch;              // value written to the flags
  int32_t region_n_tiles;      // tile columns of one owner's region (flag indexing)
  int32_t quarters;            // flags per source rank: region tiles x 4
  void* dest[CAKE_MAX_WORLD];  // per-owner base of the [out_rows, out_cols] destination
  uint32_t* flags_at[CAKE_MAX_WORLD];  // per owner: its flags for this source rank, [quarters]
  int32_t* push_done;          // kPublishAtEnd: blocks whose stores have completed; 0 between launches
  ReduceParams red;
  int32_t* status;
};

__device__ __forceinline__ void record_status(int32_t* status, int code, int d0, int d1, int d2) {
  if (status && atomicCAS(status, 0, code) == 0) {
    status[1] = d0;
    status[2] = d1;
    status[3] = d2;
  }
}

// Bounded mbarrier wait that also gives up when another role of this CTA has aborted.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity,
                                              volatile uint32_t* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag) return false;
    if (clock64() - start > kBarrierBudgetCycles) return false;
  }
}

// Grouped rasterisation: consecutive tile ids walk `rows` row-tiles down before moving one column-tile
// right, so the CTAs of one wave share A rows and B columns in L2. A wave of 148 tiles that is r
// row-tiles high touches r A panels and 148 / r B panels, a B panel being tile_n / 128 times as many
// bytes: with 128 x 256 tiles r + 296 / r is least near 17, and 16 measured 1.5 % faster than 8 on
// 8192 x 16384 x 8192 (4 rows: 5 % slower; 12: 0.8 %, 32: 0.4 % faster than 8).
__device__ __forceinline__ int raster_rows(int tile_n) { return tile_n >= 256 ? 16 : 8; }

__device__ __forceinline__ void raster(int t, int mt_count, int nt_count, int rows, int& mi, int& ni) {
  const int group_sz = rows * nt_count;
  const int g = t / group_sz;
  const int first_m = g * rows;
  const int gm = min(rows, mt_count - first_m);
  const int r = t - g * group_sz;
  mi = first_m + r % gm;
  ni = r / gm;
}

// Tile t of this rank's walk. With region_order, W consecutive tiles are the same tile of the W
// owners' regions, so every owner's region fills front to back at the pace of the whole kernel and
// link traffic is spread over all destination ports. Which owner comes first shifts by one every
// `owner_rotation` groups: a CTA's stride through the tile list (the grid size) would otherwise
// give it the same one or two owners for the whole kernel, and the CTAs that never meet their own
// (link-free) tiles would finish last.
template <int BN>
__device__ __forceinline__ void tile_coords(const MatmulParams& p, int t, int& mt, int& nt, int& owner,
                                            int& region_tile) {
  owner = 0;
  region_tile = 0;
  if (p.region_order) {
    // The walk has three parts: groups of W tiles (the same region tile of every owner, this rank's
    // included), then groups of W - 1 tiles (peers only), then the `own_tail` own tiles that were
    // left out of those groups. While the own tail is contracted nothing crosses the link, so the
    // last pushes, their arrival at the owners and the reduction that waits for this rank's own
    // partial run under that contraction instead of after the kernel's last MMA.
    const int peers = p.world - 1;
    const int mixed_groups = p.region_tiles - p.own_tail;
    const int mixed_tiles = mixed_groups * p.world;
    const int peer_tiles = p.own_tail * peers;
    int group;
    if (t < mixed_tiles) {
      group = t / p.world;
      const int j = (t - group * p.world + group / p.owner_rotation) % p.world;
      owner = (p.rank + 1 + j) % p.world;
    } else if (t < mixed_tiles + peer_tiles) {
      const int u = t - mixed_tiles;
      const int g = u / peers;
      const int j = (u - g * peers + g / p.owner_rotation) % peers;
      owner = (p.rank + 1 + j) % p.world;
      group = mixed_groups + g;
    } else {
      group = mixed_groups + (t - mixed_tiles - peer_tiles);
      owner = p.rank;
    }
    int mi, ni;
    if (p.scatter_dim == 0) {
      const int m_tiles_r = p.out_rows / kTileM;
      raster(group, m_tiles_r, p.n_tiles, raster_rows(BN), mi, ni);
      mt = owner * m_tiles_r + mi;
      nt = ni;
    } else {
      const int n_tiles_r = p.out_cols / BN;
      raster(group, p.m_tiles, n_tiles_r, raster_rows(BN), mi, ni);
      mt = mi;
      nt = owner * n_tiles_r + ni;
    }
    region_tile = mi * p.region_n_tiles + ni;
  } else {
    raster(t, p.m_tiles, p.n_tiles, raster_rows(BN), mt, nt);
  }
}

// Destination of element (r, c) of the partial: which owner, and where in its local output.
__device__ __forceinline__ char* dest_addr(const MatmulParams& p, int r, int c, int elem_bytes) {
  int owner, lr, lc;
  if (p.scatter_dim == 0) {
    owner = r / p.out_rows;
    lr = r - owner * p.out_rows;
    lc = c;
  } else {
    owner = c / p.out_cols;
    lr = r;
    lc = c - owner * p.out_cols;
  }
  return static_cast<char*>(p.dest[owner]) +
         (static_cast<size_t>(lr) * p.out_cols + lc) * static_cast<size_t>(elem_bytes);
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// ------------------------------------------------------------------------------ slot reduction

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_sys_u32(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* addr, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_cta_shared_u32(const volatile uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_u32(const_cast<const uint32_t*>(addr))) : "memory");
  return v;
}

__device__ __forceinline__ void st_release_cta_shared_u32(volatile uint32_t* addr, uint32_t v) {
  asm volatile("st.release.cta.shared.u32 [%0], %1;" ::"r"(smem_u32(const_cast<uint32_t*>(addr))), "r"(v) : "memory");
}

// Slot data is read once, after its flag has been seen: straight from L2, no L1 allocation.
__device__ __forceinline__ uint4 ld_slot_v4(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(ptr));
  return v;
}

// Waits until every source rank has announced `quarter` for this call: lane s watches source s.
// Warp-uniform result; false when the budget ran out (the status word names the first missing source).
__device__ __forceinline__ bool wait_quarter(const ReduceParams& r, int quarter, int lane,
                                             unsigned long long start, int item) {
  const uint32_t* flag = r.flags + static_cast<size_t>(lane < r.world ? lane : 0) * r.quarters + quarter;
  while (true) {
    const uint32_t seen = ld_acquire_sys_u32(flag);
    const uint32_t missing =
        __ballot_sync(0xffffffffu, lane < r.world && static_cast<int32_t>(seen - r.epoch) < 0);
    if (missing == 0) return true;
    if (__any_sync(0xffffffffu, global_timer_ns() - start > r.budget_ns)) {
      if (lane == 0) record_status(r.status, 2, blockIdx.x, __ffs(missing) - 1, item);
      return false;
    }
    __nanosleep(250);
  }
}

// One chunk = 32 rows x 128 bytes of the transport dtype (what one epilogue tensor store carries),
// reduced by one warp once its quarter has arrived. Lane l owns the 16-byte piece (l & 7) of rows
// (l >> 3) + 4 j, j = 0..7; 16 / W rows are in flight per lane at a time (16 loads of 16 bytes
// whatever the mesh size), all issued before any is used; the sum runs in rank order.
// The caller guarantees out_rows % 8 == 0, so rows j and j + 1 (j even) are inside the output together.
template <bool IN_F32, int W>
__device__ __forceinline__ void reduce_chunk_vec(const ReduceParams& r, int row0, int col0, int lane) {
  constexpr int EPP = IN_F32 ? 4 : 8;  // elements per 16-byte piece
  constexpr int TS = IN_F32 ? 4 : 2;
  constexpr int ROWS = 16 / W;
  const int col = col0 + (lane & 7) * EPP;
  if (col >= r.out_cols) return;  // the last chunk of a row may be ragged
  const size_t first = static_cast<size_t>(row0 + (lane >> 3)) * r.out_cols + col;
#pragma unroll 1
  for (int i = 0; i < 8; i += ROWS) {
    if (row0 + 4 * i >= r.out_rows) break;
    size_t offset[ROWS];
    bool active[ROWS];
    uint4 raw[ROWS][W];
#pragma unroll
    for (int u = 0; u < ROWS; ++u) {
      active[u] = row0 + 4 * ((i + u) & ~1) < r.out_rows;
      // A row outside the output re-reads the chunk's first row (in bounds, no predicate needed).
      offset[u] = active[u] ? first + static_cast<size_t>(4 * (i + u)) * r.out_cols : first;
#pragma unroll
      for (int src = 0; src < W; ++src) raw[u][src] = ld_slot_v4(r.slots + src * r.slot_stride + offset[u] * TS);
    }
#pragma unroll
    for (int u = 0; u < ROWS; ++u) {
      if (!active[u]) continue;
      float acc[EPP];
#pragma unroll
      for (int e = 0; e < EPP; ++e) acc[e] = 0.f;
#pragma unroll
      for (int src = 0; src < W; ++src) {
        const uint4 v = raw[u][src];
        if (IN_F32) {
          acc[0] += __uint_as_float(v.x);
          acc[1] += __uint_as_float(v.y);
          acc[2] += __uint_as_float(v.z);
          acc[3] += __uint_as_float(v.w);
        } else {
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            acc[2 * e] += __uint_as_float(w[e] << 16);
            acc[2 * e + 1] += __uint_as_float(w[e] & 0xFFFF0000u);
          }
        }
      }
      if (r.out_f32) {
        float* dst = static_cast<float*>(r.out) + offset[u];
#pragma unroll
        for (int e = 0; e < EPP; e += 4)
          *reinterpret_cast<float4*>(dst + e) = make_float4(acc[e], acc[e + 1], acc[e + 2], acc[e + 3]);
      } else if (EPP == 8) {
        uint4 packed;
        packed.x = pack2_bf16(acc[0], acc[1]);
        packed.y = pack2_bf16(acc[2], acc[3]);
        packed.z = pack2_bf16(acc[4], acc[5]);
        packed.w = pack2_bf16(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(r.out) + offset[u]) = packed;
      } else {
        uint2 packed;
        packed.x = pack2_bf16(acc[0], acc[1]);
        packed.y = pack2_bf16(acc[2], acc[3]);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(r.out) + offset[u]) = packed;
      }
    }
  }
}

template <bool IN_F32>
__device__ __forceinline__ void reduce_chunk_vec_world(const ReduceParams& r, int row0, int col0, int lane) {
  if (r.world == 8) reduce_chunk_vec<IN_F32, 8>(r, row0, col0, lane);
  else if (r.world == 4) reduce_chunk_vec<IN_F32, 4>(r, row0, col0, lane);
  else reduce_chunk_vec<IN_F32, 2>(r, row0, col0, lane);
}

// The same chunk element by element, for shapes the vector path does not cover.
__device__ __forceinline__ void reduce_chunk_scalar(const ReduceParams& r, int row0, int col0, int lane) {
  const int ts = r.in_f32 ? 4 : 2;
  const int cols_per_chunk = 128 / ts;
  for (int idx = lane; idx < 32 * cols_per_chunk; idx += 32) {
    const int row = row0 + idx / cols_per_chunk;
    const int col = col0 + idx % cols_per_chunk;
    if (row >= r.out_rows || col >= r.out_cols) continue;
    const size_t offset = static_cast<size_t>(row) * r.out_cols + col;
    float acc = 0.f;
    for (int src = 0; src < r.world; ++src) {
      const char* piece = r.slots + src * r.slot_stride + offset * ts;
      const uint32_t v = r.in_f32 ? __ldcg(reinterpret_cast<const uint32_t*>(piece))
                                  : static_cast<uint32_t>(__ldcg(reinterpret_cast<const uint16_t*>(piece))) << 16;
      acc += __uint_as_float(v);
    }
    if (r.out_f32) static_cast<float*>(r.out)[offset] = acc;
    else static_cast<__nv_bfloat16*>(r.out)[offset] = __float2bfloat16_rn(acc);
  }
}

// One reduction worker (a whole warp). Chunks are numbered in the order the pushing side produces
// them -- tiles of 128 x tile_n in the raster order of tile_coords, then the four 32-row quarters,
// then the 128-byte column chunks -- and handed out through a ticket counter, so whichever warps
// are free take the next chunk to arrive: the dedicated reduction warps during the contraction,
// and every warp of the kernel once its own role is done, which keeps the tail after the last
// tile short. The next ticket is drawn before the current chunk is worked on.
__device__ __forceinline__ void reduce_worker(const ReduceParams& r, int lane) {
  const int cols_per_chunk = r.in_f32 ? 32 : 64;
  const int chunks_per_quarter = r.tile_n / cols_per_chunk;
  const int m_tiles = (r.out_rows + kTileM - 1) / kTileM;
  const int n_tiles = (r.out_cols + r.tile_n - 1) / r.tile_n;
  const int items = m_tiles * n_tiles * 4 * chunks_per_quarter;
  const unsigned long long start = global_timer_ns();
  int next = 0;
  if (lane == 0) next = atomicAdd(r.tickets, 1);
  while (true) {
    const int item = __shfl_sync(0xffffffffu, next, 0);
    if (item >= items) break;
    if (lane == 0) next = atomicAdd(r.tickets, 1);
    const int tile = item / (4 * chunks_per_quarter);
    const int rest = item - tile * 4 * chunks_per_quarter;
    const int q = rest / chunks_per_quarter;
    int mi, ni;
    raster(tile, m_tiles, n_tiles, raster_rows(r.tile_n), mi, ni);
    const int row0 = mi * kTileM + q * 32;
    const int col0 = ni * r.tile_n + (rest - q * chunks_per_quarter) * cols_per_chunk;
    if (row0 >= r.out_rows || col0 >= r.out_cols) continue;
    if (!wait_quarter(r, (mi * n_tiles + ni) * 4 + q, lane, start, item)) break;
    if (!r.vec_ok) reduce_chunk_scalar(r, row0, col0, lane);
    else if (r.in_f32) reduce_chunk_vec_world<true>(r, row0, col0, lane);
    else reduce_chunk_vec_world<false>(r, row0, col0, lane);
  }
}

// Called by one thread of every block after the block's last worker has left reduce_worker: the
// last block to get here puts the ticket counter back to zero for the next launch.
__device__ __forceinline__ void reduce_block_done(const ReduceParams& r) {
  __threadfence();
  if (atomicAdd(r.tickets + 1, 1) == static_cast<int>(gridDim.x) - 1) {
    r.tickets[0] = 0;
    r.tickets[1] = 0;
    __threadfence();
  }
}

// The slot reduction as a kernel of its own.
__global__ void __launch_bounds__(256) cake_reduce_slots_sm100(const __grid_constant__ ReduceParams r) {
  reduce_worker(r, threadIdx.x & 31);
  __syncthreads();
  if (threadIdx.x == 0) reduce_block_done(r);
}

// cp.async.bulk.wait_group takes its count as an immediate.
__device__ __forceinline__ void bulk_wait_group_at_most(int pending) {
  switch (pending) {
    case 0: asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); break;
    case 1: asm volatile("cp.async.bulk.wait_group 1;" ::: "memory"); break;
    case 2: asm volatile("cp.async.bulk.wait_group 2;" ::: "memory"); break;
    case 4: asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); break;
    default: asm volatile("cp.async.bulk.wait_group 8;" ::: "memory"); break;
  }
}

// One tensor map per owner: its [out_rows, out_cols] destination (own output, owner-major partial or
// a peer's receive slot), boxes of 32 rows x 128 bytes, 128-byte swizzle.
struct OwnerMaps {
  CUtensorMap m[CAKE_MAX_WORLD];
};

template <int BN, bool B_KMAJOR>
__global__ void __launch_bounds__(kGemmThreads, 1)
    cake_matmul_rs_sm100(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ OwnerMaps owner_maps,
                         const __grid_constant__ MatmulParams p) {
  using Cfg = GemmCfg<BN>;
  constexpr int STAGES = Cfg::kStages;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* staging = smem + STAGES * Cfg::kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + 4 * kStagingBytesPerWarp);
  uint64_t* full_bar = bars;                 // [STAGES]
  uint64_t* empty_bar = bars + STAGES;       // [STAGES]
  uint64_t* tmem_full = bars + 2 * STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;      // [2]
  uint64_t* drain_bar = tmem_empty + 2;      // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  volatile uint32_t* epilogue_done = tmem_base_slot + 2;  // epilogue warps whose stores have completed
  // Mailbox between the epilogue warps and the publisher warp: what epilogue warp i has handed over
  // so far (with kMailDone once it has finished), what the publisher has sent of it, and the ring of
  // announcements in between, each packed as owner << 24 | flag index.
  volatile uint32_t* mail_seq = tmem_base_slot + 4;     // [4]
  volatile uint32_t* mail_taken = mail_seq + 4;         // [4]
  volatile uint32_t* mail_ring = mail_taken + 4;        // [4][kMailDepth]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.m_tiles * p.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&tmem_full[b]), 1);
      mbar_init(smem_u32(&tmem_empty[b]), 4);
    }
    mbar_init(smem_u32(drain_bar), 1);
    *abort_flag = 0;
    *epilogue_done = 0;
    for (int i = 0; i < 4; ++i) {
      mail_seq[i] = 0;
      mail_taken[i] = 0;
    }
    fence_mbar_init();
    prefetch_tensormap(&tmap_a);
    prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_base_slot), Cfg::kTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int mt, nt, owner_unused, region_unused;
        tile_coords<BN>(p, t, mt, nt, owner_unused, region_unused);
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!wait_or_abort(smem_u32(&empty_bar[stage]), phase ^ 1, abort_flag)) {
            if (!*abort_flag) record_status(p.status, 1, blockIdx.x, t, 100 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&full_bar[stage]);
          const uint32_t a_dst = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t b_dst = a_dst + kABytes;
          mbar_arrive_expect_tx(full, Cfg::kStageBytes);
          tma_load_2d(a_dst, &tmap_a, full, kb * kBlockK, mt * kTileM);
          if (B_KMAJOR) {
            tma_load_2d(b_dst, &tmap_b, full, kb * kBlockK, nt * BN);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) {
              tma_load_2d(b_dst + j * (64 * kBlockK * 2), &tmap_b, full, nt * BN + j * 64,
                          kb * kBlockK);
            }
          }
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Let copies already in flight land before the CTA's shared memory is released.
        for (int s = 0; s < STAGES; ++s) {
          const uint32_t par = (s < stage) ? phase : (phase ^ 1);
          mbar_wait_bounded(smem_u32(&full_bar[s]), par, 200000000ll);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16_f32(kTileM, BN, 0, B_KMAJOR ? 0 : 1);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1;
        if (!wait_or_abort(smem_u32(&tmem_empty[buf]), acc_phase ^ 1, abort_flag)) {
          if (!*abort_flag) record_status(p.status, 1, blockIdx.x, t, 200 + buf);
          *abort_flag = 1;
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!wait_or_abort(smem_u32(&full_bar[stage]), phase, abort_flag)) {
            if (!*abort_flag) record_status(p.status, 1, blockIdx.x, t, 300 + stage);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * Cfg::kStageBytes);
          const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
          for (int kk = 0; kk < kBlockK / kUmmaK; ++kk) {
            // A (K-major): 8-row groups 1024 B apart; a K step of 16 elements is 32 B inside the
            // 128-byte swizzle row.
            const uint64_t a_desc = umma_desc_sw128(a_addr + kk * 32, 16, 1024);
            // B as [N,K] (K-major): same as A. B as [K,N] (MN-major): 64-column blocks 8192 B
            // apart (leading offset), 8-deep K groups 1024 B apart (stride offset); a K step of
            // 16 is two such groups.
            const uint64_t b_desc = B_KMAJOR ? umma_desc_sw128(b_addr + kk * 32, 16, 1024)
                                             : umma_desc_sw128(b_addr + kk * 2048, 8192, 1024);
            tcgen05_mma_bf16(tmem_d, a_desc, b_desc, idesc, (kb | kk) != 0 ? 1u : 0u);
          }
          tcgen05_commit(smem_u32(&empty_bar[stage]));
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tcgen05_commit(smem_u32(&tmem_full[buf]));
      }
      // Drain: every MMA issued above has retired before TMEM is released.
      tcgen05_commit(smem_u32(drain_bar));
      mbar_wait_bounded(smem_u32(drain_bar), 0, kBarrierBudgetCycles);
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ epilogue warps 2..5
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    uint8_t* my_stage_base = staging + (warp - 2) * kStagingBytesPerWarp;
    int chunk_count = 0;  // chunks this warp has staged so far (selects the staging half)
    uint32_t* pending_flag = nullptr;  // lane 0: the flag of the quarter sent last, not yet announced
    uint32_t pending_packed = 0;       // the same flag as owner << 24 | index, for the mailbox
    uint32_t handed = 0;               // announcements handed to the publisher warp so far
    // A release store at system scope holds its thread until the SM's earlier writes have been
    // acknowledged from across the link; issued here once per tile it cost a fifth of the push rate
    // (4 GPUs pushing 4 KiB tensor stores from 4 warps per SM: 644 GB/s per GPU, 502 with the release
    // store, 644 again with a relaxed one). So the epilogue warp only waits for its stores, fences
    // the proxy and hands the flag over through shared memory; the publisher warp issues the release.
    auto announce = [&](bool last) {
      if (!p.mailbox) {
        if (pending_flag != nullptr) st_release_sys_u32(pending_flag, p.epoch);
        return;
      }
      const int w = warp - 2;
      if (pending_flag != nullptr) {
        if (handed - ld_acquire_cta_shared_u32(mail_taken + w) >= kMailDepth) {
          const long long start = clock64();
          while (handed - ld_acquire_cta_shared_u32(mail_taken + w) >= kMailDepth) {
            if (*abort_flag || clock64() - start > kBarrierBudgetCycles) {
              if (!*abort_flag) record_status(p.status, 1, blockIdx.x, static_cast<int>(handed), 500 + w);
              *abort_flag = 1;
              return;
            }
          }
        }
        mail_ring[w * kMailDepth + handed % kMailDepth] = pending_packed;
        ++handed;
      }
      st_release_cta_shared_u32(mail_seq + w, handed | (last ? kMailDone : 0u));
    };
    const int elem_bytes = p.store_f32 ? 4 : 2;
    const int cols_per_chunk = p.store_f32 ? 32 : 64;  // 128 bytes per row per chunk
    const int epp = 16 / elem_bytes;                   // elements per 16-byte piece
    int it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++it) {
      int mt, nt, owner, region_tile;
      tile_coords<BN>(p, t, mt, nt, owner, region_tile);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1;
      // The decision is made warp-uniform: tcgen05.ld below is a warp-collective instruction.
      if (!__all_sync(0xffffffffu, wait_or_abort(smem_u32(&tmem_full[buf]), acc_phase, abort_flag))) {
        if (!*abort_flag && lane == 0) record_status(p.status, 1, blockIdx.x, t, 400 + buf);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN;
      const int row0 = mt * kTileM + q * 32;
      const int num_chunks = BN / cols_per_chunk;
      for (int ch = 0; ch < num_chunks; ++ch) {
        uint4 pieces[8];
        if (p.store_f32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(t_row + ch * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            pieces[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_row + ch * 64 + h * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[8 * j + 2 * e]),
                                                                __uint_as_float(v[8 * j + 2 * e + 1]));
                w[e] = *reinterpret_cast<const uint32_t*>(&b2);
              }
              pieces[h * 4 + j] = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
        }
        if (ch == num_chunks - 1) {
          // The accumulator buffer is fully read: hand it back to the MMA warp.
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&tmem_empty[buf]));
        }
        // Transpose through swizzled smem (the layout of a 128-byte-swizzled TMA box) so that the
        // chunk leaves as 128-byte row segments.
        uint8_t* my_stage = my_stage_base + (chunk_count % kStagingChunks) * (32 * 128);
        if (p.tma_store && chunk_count >= kStagingChunks) {
          // A staging slot is reused every kStagingChunks chunks: its previous store must have read it.
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kStagingChunks - 1) : "memory");
          __syncwarp();
        }
        ++chunk_count;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          *reinterpret_cast<uint4*>(my_stage + lane * 128 + ((j ^ (lane & 7)) << 4)) = pieces[j];
        }
        if (p.tma_store) {
          fence_proxy_async_smem();  // generic-proxy writes above -> visible to the TMA engine
          __syncwarp();
          const int r = row0;
          const int c = nt * BN + ch * cols_per_chunk;
          if (lane == 0 && r < p.m && c < p.n) {
            int owner, lr, lc;
            if (p.scatter_dim == 0) {
              owner = r / p.out_rows;
              lr = r - owner * p.out_rows;
              lc = c;
            } else {
              owner = c / p.out_cols;
              lr = r;
              lc = c - owner * p.out_cols;
            }
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                         ::"l"(reinterpret_cast<uint64_t>(&owner_maps.m[owner])), "r"(smem_u32(my_stage)),
                         "r"(lc), "r"(lr)
                         : "memory");
          }
          if (lane == 0) asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          continue;
        }
        __syncwarp();
        const int pj = lane & 7;
        const int c = nt * BN + ch * cols_per_chunk + pj * epp;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int rr = i * 4 + (lane >> 3);
          const int r = row0 + rr;
          const uint4 val = *reinterpret_cast<const uint4*>(my_stage + rr * 128 + ((pj ^ (rr & 7)) << 4));
          if (r < p.m) {
            if (p.vec_ok) {
              if (c < p.n) *reinterpret_cast<uint4*>(dest_addr(p, r, c, elem_bytes)) = val;
            } else if (p.store_f32) {
              const uint32_t w[4] = {val.x, val.y, val.z, val.w};
              for (int e = 0; e < 4; ++e)
                if (c + e < p.n)
                  *reinterpret_cast<uint32_t*>(dest_addr(p, r, c + e, 4)) = w[e];
            } else {
              const uint32_t w[4] = {val.x, val.y, val.z, val.w};
              for (int e = 0; e < 8; ++e)
                if (c + e < p.n)
                  *reinterpret_cast<uint16_t*>(dest_addr(p, r, c + e, 2)) =
                      static_cast<uint16_t>(w[e >> 1] >> ((e & 1) * 16));
            }
          }
        }
        __syncwarp();
      }
      if (p.publish == kPublishPerTile && lane == 0) {
        // Announce the quarter sent one tile ago: its stores were issued a whole main loop ago, so
        // waiting for all but this tile's groups costs nothing. Completion of a bulk group makes
        // its writes visible to this thread; the proxy fence orders them before the release store.
        // A quarter of the rank's own region is announced at once: its stores are local and complete
        // in about a microsecond, and the reduction of that tile need not wait a whole main loop.
        const bool now = p.own_now && owner == p.rank;
        if (pending_flag != nullptr || now) {
          bulk_wait_group_at_most(now ? 0 : num_chunks);
          asm volatile("fence.proxy.async.global;" ::: "memory");
          if (pending_flag != nullptr) announce(false);
        }
        pending_flag = p.flags_at[owner] + region_tile * 4 + (warp - 2);
        pending_packed = (static_cast<uint32_t>(owner) << 24) | static_cast<uint32_t>(region_tile * 4 + (warp - 2));
        if (now) {
          announce(false);
          pending_flag = nullptr;
        }
      }
    }
    if (p.publish == kPublishPerTile && lane == 0) {
      // The last quarter, and the word that lets the publisher warp leave (also when this warp gave up).
      if (!ok) pending_flag = nullptr;
      if (pending_flag != nullptr) {
        bulk_wait_group_at_most(0);
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      announce(true);
    }
    if (p.publish == kPublishAtEnd && ok) {
      // Tiles may straddle owners here, so nothing is announced per tile: every epilogue warp
      // makes its own stores visible, the block's last warp counts the block as done, and the
      // last block of the grid announces every quarter to every owner.
      __syncwarp();
      int last_block = 0;
      if (lane == 0) {
        if (p.tma_store) {
          bulk_wait_group_at_most(0);
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        __threadfence_system();
        if (atomicAdd(const_cast<uint32_t*>(epilogue_done), 1u) == 3u) {
          __threadfence_system();
          last_block = atomicAdd(p.push_done, 1) == static_cast<int>(gridDim.x) - 1;
        }
      }
      last_block = __shfl_sync(0xffffffffu, last_block, 0);
      if (last_block) {
        __threadfence_system();
        for (int o = 0; o < p.world; ++o)
          for (int idx = lane; idx < p.quarters; idx += 32) st_release_sys_u32(p.flags_at[o] + idx, p.epoch);
        if (lane == 0) *p.push_done = 0;
      }
    }
  }
  else if (warp == kPublisherWarp && p.publish == kPublishPerTile && p.mailbox) {
    // ------------------------------------------------------------------ publisher
    // Lane i < 4 serves epilogue warp i: whatever it has handed over since the last look is
    // announced behind one system-scope fence (fence + relaxed stores form the release), so the
    // wait for the acknowledgements is spent by a warp that has nothing else to do.
    uint32_t taken = 0;
    long long start = clock64();
    while (true) {
      const uint32_t word = lane < 4 ? ld_acquire_cta_shared_u32(mail_seq + lane) : kMailDone;
      const uint32_t avail = word & ~kMailDone;
      const bool have = lane < 4 && avail != taken;
      if (have) {
        asm volatile("fence.acq_rel.sys;" ::: "memory");
        while (taken != avail) {
          const uint32_t packed = mail_ring[lane * kMailDepth + taken % kMailDepth];
          st_relaxed_sys_u32(p.flags_at[packed >> 24] + (packed & 0xFFFFFFu), p.epoch);
          ++taken;
        }
        st_release_cta_shared_u32(mail_taken + lane, taken);
      }
      if (__all_sync(0xffffffffu, (word & kMailDone) != 0 && !have)) break;
      if (*abort_flag) break;
      if (__any_sync(0xffffffffu, have)) {
        start = clock64();
      } else if (clock64() - start > kBarrierBudgetCycles) {
        if (lane == 0 && !*abort_flag) record_status(p.status, 1, blockIdx.x, static_cast<int>(taken), 600);
        *abort_flag = 1;
        break;
      } else {
        __nanosleep(64);
      }
    }
  }
  // ------------------------------------------------------------------ slot reduction
  // Warps 6..10 do nothing else; the publisher and the others join when their own role is done (unless the block has
  // given up on one of its barriers), so the chunks that arrive last find every warp free.
  __syncwarp();
  if (p.reduce_in_kernel && !*abort_flag) reduce_worker(p.red, lane);

  // Shared memory must outlive every tensor store that still reads it.
  if (p.tma_store && warp >= 2 && warp < 6 && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  if (p.reduce_in_kernel && threadIdx.x == 0) reduce_block_done(p.red);
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::kTmemCols);
}

// bf16 [rows, cols] -> [cols, rows]; used only when the caller asks the library to consume the
// reference's [K,N] rhs through the K-major operand path.
__global__ void cake_transpose_bf16(const uint16_t* __restrict__ in, uint16_t* __restrict__ out,
                                    int rows, int cols) {
  __shared__ uint16_t tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int r = r0 + i, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[i][threadIdx.x] = in[static_cast<size_t>(r) * cols + c];
  }
  __syncthreads();
  for (int i = threadIdx.y; i < 32; i += blockDim.y) {
    const int c = c0 + i, r = r0 + threadIdx.x;
    if (r < rows && c < cols) out[static_cast<size_t>(c) * rows + r] = tile[threadIdx.x][i];
  }
}

}  // namespace cake

// ====================================================================================== host

struct cake_matmul_rs {
  cake_matmul_rs_desc d;
  int device = 0;
  int sm_count = 0;
  int64_t out_rows = 0, out_cols = 0;
  size_t tsize = 4;  // bytes per transported element
  size_t osize = 4;  // bytes per output element
  bool rhs_via_transpose = false;
  void* rhs_t = nullptr;  // [n, k_local] scratch when rhs_via_transpose
  void* slots[CAKE_MAX_WORLD] = {};
  void* flags[CAKE_MAX_WORLD] = {};
  size_t slot_stride = 0;  // bytes between two sources' slots: one local output, padded to 128 bytes
  int region_m_tiles = 0, region_n_tiles = 0;  // tile grid of one owner's region
  int quarters = 0;                            // arrival flags per source rank
  int32_t* tickets = nullptr;  // 3 x int32 on the device: chunk ticket, reduction blocks done, push blocks done
  bool bound = false;
  unsigned long long epoch = 0;
  cake::StatusWord status;
  // tensor-map cache
  const void* last_lhs = nullptr;
  const void* last_rhs = nullptr;
  CUtensorMap tmap_a, tmap_b;
  cake::OwnerMaps owner_maps[2];  // per slot parity (index 0 also serves the non-peer modes)
  const void* owner_maps_base[2] = {nullptr, nullptr};
  // staging for run_host
  void* h_lhs = nullptr;
  void* h_rhs = nullptr;
  void* h_out = nullptr;
  // run_host at world 1: a plan for one block of rows, and what overlaps the copies with it
  static constexpr int kHostBlocks = 8;
  cake_matmul_rs* row_block_plan = nullptr;
  int host_blocks = 0;  // 0 = not decided yet, 1 = one enqueue for the whole matrix
  cudaStream_t copy_in = nullptr, copy_out = nullptr;
  cudaEvent_t host_begin = nullptr, host_end = nullptr;
  cudaEvent_t block_in[kHostBlocks] = {}, block_done[kHostBlocks] = {};
  int launches = 0;
};

namespace {

using cake::fail;

template <int BN, bool KM>
int32_t launch_gemm(const cake_matmul_rs* plan, const cake::MatmulParams& p, int grid,
                    cudaStream_t stream, int maps_index) {
  auto kernel = cake::cake_matmul_rs_sm100<BN, KM>;
  // The opt-in to more than 48 KB of dynamic shared memory is a per-device attribute.
  static bool configured[64] = {};
  const int slot = plan->device >= 0 && plan->device < 64 ? plan->device : 0;
  if (!configured[slot]) {
    CAKE_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       cake::GemmCfg<BN>::kSmemBytes));
    configured[slot] = plan->device >= 0 && plan->device < 64;
  }
  kernel<<<grid, cake::kGemmThreads, cake::GemmCfg<BN>::kSmemBytes, stream>>>(
      plan->tmap_a, plan->tmap_b, plan->owner_maps[maps_index], p);
  CAKE_CUDA_TRY(cudaGetLastError());
  return CAKE_OK;
}

int32_t encode_maps(cake_matmul_rs* plan, const void* lhs, const void* rhs_kmajor_or_mn) {
  const cake_matmul_rs_desc& d = plan->d;
  const bool kmajor = d.rhs_layout == 1 || plan->rhs_via_transpose;
  {
    const uint64_t dims[2] = {static_cast<uint64_t>(d.k_local), static_cast<uint64_t>(d.m)};
    const uint64_t strides[1] = {static_cast<uint64_t>(d.k_local) * 2};
    const uint32_t box[2] = {cake::kBlockK, cake::kTileM};
    int32_t rc = cake::encode_tensor_map(&plan->tmap_a, lhs, 2, dims, strides, box, true);
    if (rc) return rc;
  }
  if (kmajor) {
    const uint64_t dims[2] = {static_cast<uint64_t>(d.k_local), static_cast<uint64_t>(d.n)};
    const uint64_t strides[1] = {static_cast<uint64_t>(d.k_local) * 2};
    const uint32_t box[2] = {cake::kBlockK, static_cast<uint32_t>(d.tile_n)};
    return cake::encode_tensor_map(&plan->tmap_b, rhs_kmajor_or_mn, 2, dims, strides, box, true);
  }
  const uint64_t dims[2] = {static_cast<uint64_t>(d.n), static_cast<uint64_t>(d.k_local)};
  const uint64_t strides[1] = {static_cast<uint64_t>(d.n) * 2};
  const uint32_t box[2] = {64, cake::kBlockK};
  return cake::encode_tensor_map(&plan->tmap_b, rhs_kmajor_or_mn, 2, dims, strides, box, true);
}

}  // namespace

extern "C" {

int32_t cake_matmul_rs_create(const cake_matmul_rs_desc* desc, cake_matmul_rs** out) {
  if (!desc || !out) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_matmul_rs_create: null argument");
  const cake_matmul_rs_desc& d = *desc;
  if (d.m <= 0 || d.n <= 0 || d.k_local <= 0 || d.m > INT32_MAX || d.n > INT32_MAX ||
      d.k_local > INT32_MAX)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "matmul shape must be positive and fit int32: m=%lld n=%lld k_local=%lld",
                (long long)d.m, (long long)d.n, (long long)d.k_local);
  if (d.world < 1 || d.world > CAKE_MAX_WORLD || d.rank < 0 || d.rank >= d.world)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "bad mesh: world=%d rank=%d", d.world, d.rank);
  if (d.scatter_dim != 0 && d.scatter_dim != 1)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "scatter_dim must be 0 (M) or 1 (N), got %d", d.scatter_dim);
  if ((d.out_dtype != CAKE_DTYPE_F32 && d.out_dtype != CAKE_DTYPE_BF16) ||
      (d.transport_dtype != CAKE_DTYPE_F32 && d.transport_dtype != CAKE_DTYPE_BF16))
    return fail(CAKE_ERR_INVALID_ARGUMENT, "out_dtype / transport_dtype must be CAKE_DTYPE_F32 or CAKE_DTYPE_BF16");
  if (d.tile_m != 128)
    return fail(CAKE_ERR_UNSUPPORTED, "tile_m must be 128 on sm_100a (UMMA M), got %d", d.tile_m);
  if (d.tile_n != 64 && d.tile_n != 128 && d.tile_n != 256)
    return fail(CAKE_ERR_UNSUPPORTED, "tile_n must be 64, 128 or 256, got %d", d.tile_n);
  if (d.k_local % 8 != 0)
    return fail(CAKE_ERR_UNSUPPORTED, "k_local must be a multiple of 8 (16-byte TMA row pitch), got %lld",
                (long long)d.k_local);
  if (d.rhs_layout == 0 && d.n % 8 != 0)
    return fail(CAKE_ERR_UNSUPPORTED, "n must be a multiple of 8 for a [k,n] rhs, got %lld", (long long)d.n);
  if (d.rhs_layout != 0 && d.rhs_layout != 1)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rhs_layout must be 0 or 1");
  const int64_t scattered = d.scatter_dim == 0 ? d.m : d.n;
  if (scattered % d.world != 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "scatter dimension %lld is not divisible by world %d",
                (long long)scattered, d.world);
  if (d.world > 1 && d.strategy != CAKE_RS_LOCAL_PARTIAL && d.strategy != CAKE_RS_P2P_OWNER_PUSH)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "unknown reduce-scatter strategy %d", d.strategy);
  if (d.wait_budget_ms < 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "wait_budget_ms must be >= 0 (0 = default), got %d", d.wait_budget_ms);

  cake_matmul_rs* plan = new (std::nothrow) cake_matmul_rs();
  if (!plan) return fail(CAKE_ERR_CUDA, "out of host memory");
  plan->d = d;
  cudaError_t e = cudaGetDevice(&plan->device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&plan->sm_count, cudaDevAttrMultiProcessorCount, plan->device);
  int major = 0;
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, plan->device);
  if (e != cudaSuccess) {
    delete plan;
    return fail(CAKE_ERR_CUDA, "no usable CUDA device: %s", cudaGetErrorString(e));
  }
  if (major != 10) {
    delete plan;
    return fail(CAKE_ERR_UNSUPPORTED, "libcake_b200 needs an sm_100 GPU, found compute capability %d.x", major);
  }
  plan->out_rows = d.scatter_dim == 0 ? d.m / d.world : d.m;
  plan->out_cols = d.scatter_dim == 1 ? d.n / d.world : d.n;
  plan->osize = d.out_dtype == CAKE_DTYPE_F32 ? 4 : 2;
  plan->tsize = d.world == 1 ? plan->osize : (d.transport_dtype == CAKE_DTYPE_F32 ? 4 : 2);
  plan->slot_stride = (static_cast<size_t>(plan->out_rows) * plan->out_cols * plan->tsize + 127) / 128 * 128;
  plan->region_m_tiles = (int)((plan->out_rows + cake::kTileM - 1) / cake::kTileM);
  plan->region_n_tiles = (int)((plan->out_cols + d.tile_n - 1) / d.tile_n);
  plan->quarters = plan->region_m_tiles * plan->region_n_tiles * 4;
  const char* env = getenv("CAKE_MATMUL_TRANSPOSE_RHS");
  plan->rhs_via_transpose = d.rhs_layout == 0 && env && env[0] == '1';
  int32_t rc = plan->status.ensure();
  if (rc == CAKE_OK && d.world > 1 && d.strategy == CAKE_RS_P2P_OWNER_PUSH) {
    e = cudaMalloc(&plan->tickets, 3 * sizeof(int32_t));
    if (e == cudaSuccess) e = cudaMemset(plan->tickets, 0, 3 * sizeof(int32_t));
    if (e != cudaSuccess) rc = fail(CAKE_ERR_CUDA, "cudaMalloc(tickets) failed: %s", cudaGetErrorString(e));
  }
  if (rc == CAKE_OK && plan->rhs_via_transpose) {
    e = cudaMalloc(&plan->rhs_t, static_cast<size_t>(d.n) * d.k_local * 2);
    if (e != cudaSuccess) rc = fail(CAKE_ERR_CUDA, "cudaMalloc(rhs_t) failed: %s", cudaGetErrorString(e));
  }
  if (rc != CAKE_OK) {
    cake_matmul_rs_destroy(plan);
    return rc;
  }
  *out = plan;
  return CAKE_OK;
}

int32_t cake_matmul_rs_destroy(cake_matmul_rs* plan) {
  if (!plan) return CAKE_OK;
  plan->status.release();
  if (plan->tickets) cudaFree(plan->tickets);
  if (plan->rhs_t) cudaFree(plan->rhs_t);
  if (plan->h_lhs) cudaFree(plan->h_lhs);
  if (plan->h_rhs) cudaFree(plan->h_rhs);
  if (plan->h_out) cudaFree(plan->h_out);
  if (plan->row_block_plan) cake_matmul_rs_destroy(plan->row_block_plan);
  if (plan->copy_in) cudaStreamDestroy(plan->copy_in);
  if (plan->copy_out) cudaStreamDestroy(plan->copy_out);
  if (plan->host_begin) cudaEventDestroy(plan->host_begin);
  if (plan->host_end) cudaEventDestroy(plan->host_end);
  for (int i = 0; i < cake_matmul_rs::kHostBlocks; ++i) {
    if (plan->block_in[i]) cudaEventDestroy(plan->block_in[i]);
    if (plan->block_done[i]) cudaEventDestroy(plan->block_done[i]);
  }
  delete plan;
  return CAKE_OK;
}

size_t cake_matmul_rs_partial_bytes(const cake_matmul_rs* plan) {
  return plan ? static_cast<size_t>(plan->d.m) * plan->d.n * plan->tsize : 0;
}

size_t cake_matmul_rs_slot_bytes(const cake_matmul_rs* plan) {
  if (!plan || plan->d.world == 1) return 0;
  // two parities x W sources x one local output in the transport dtype (padded to 128 bytes)
  return 2ull * plan->d.world * plan->slot_stride;
}

size_t cake_matmul_rs_flag_bytes(const cake_matmul_rs* plan) {
  if (!plan || plan->d.world == 1) return 0;
  // one 32-bit call number per source rank and quarter tile
  return (static_cast<size_t>(plan->d.world) * plan->quarters * sizeof(uint32_t) + 127) / 128 * 128;
}

int32_t cake_matmul_rs_bind_peers(cake_matmul_rs* plan, void* const* slots, void* const* flags) {
  if (!plan || !slots || !flags) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_matmul_rs_bind_peers: null argument");
  for (int r = 0; r < plan->d.world; ++r) {
    if (!slots[r] || !flags[r]) return fail(CAKE_ERR_INVALID_ARGUMENT, "missing slot/flag pointer for rank %d", r);
    if ((reinterpret_cast<uintptr_t>(slots[r]) & 127) || (reinterpret_cast<uintptr_t>(flags[r]) & 3))
      return fail(CAKE_ERR_INVALID_ARGUMENT, "slot pointer of rank %d must be 128-byte aligned, flags 4-byte aligned", r);
    plan->slots[r] = slots[r];
    plan->flags[r] = flags[r];
  }
  plan->bound = true;
  return CAKE_OK;
}

int32_t cake_matmul_rs_launches_per_enqueue(const cake_matmul_rs* plan) { return plan ? plan->launches : 0; }

}  // extern "C"

namespace {
constexpr int kPhasePush = 1;    // contraction + epilogue stores / pushes
constexpr int kPhaseReduce = 2;  // slot reduction (peer-to-peer strategy only)

// Fills the reduction's parameters for the slots of `parity`.
void fill_reduce_params(const cake_matmul_rs* plan, unsigned long long parity, void* out,
                        cake::ReduceParams* r) {
  const cake_matmul_rs_desc& d = plan->d;
  r->slots = static_cast<const char*>(plan->slots[d.rank]) + parity * d.world * plan->slot_stride;
  r->flags = static_cast<const uint32_t*>(plan->flags[d.rank]);
  r->epoch = static_cast<uint32_t>(plan->epoch);
  r->quarters = plan->quarters;
  r->out = out;
  r->slot_stride = plan->slot_stride;
  const unsigned long long ms = d.wait_budget_ms > 0 ? static_cast<unsigned long long>(d.wait_budget_ms)
                                                     : cake::kDefaultPeerBudgetMs;
  r->budget_ns = ms * 1000000ull;
  r->out_rows = (int)plan->out_rows;
  r->out_cols = (int)plan->out_cols;
  r->world = d.world;
  r->in_f32 = plan->tsize == 4;
  r->out_f32 = plan->osize == 4;
  // The vector path wants whole 16-byte pieces per row in the transport dtype (the output row then
  // is a whole number of 8-byte (bf16 out of f32) to 32-byte (f32 out of bf16) pieces of a 16-byte
  // aligned base), rows in whole groups of 8, and a mesh of 2, 4 or 8; anything else goes element
  // by element.
  r->vec_ok = plan->out_cols % (16 / (int)plan->tsize) == 0 && plan->out_rows % 8 == 0 &&
              (d.world == 2 || d.world == 4 || d.world == 8);
  r->tile_n = d.tile_n;
  r->tickets = plan->tickets;
  r->status = plan->status.dev;
}

int32_t enqueue_impl(cake_matmul_rs* plan, const void* lhs, const void* rhs, void* out,
                     void* stream_v, int phases) {
  if (!plan || !out) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_matmul_rs_enqueue: null argument");
  if ((phases & kPhasePush) && (!lhs || !rhs)) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_matmul_rs_enqueue: null operand");
  const cake_matmul_rs_desc& d = plan->d;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if ((reinterpret_cast<uintptr_t>(lhs) | reinterpret_cast<uintptr_t>(rhs) |
       reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "lhs, rhs and out must be 16-byte aligned");
  const bool p2p = d.world > 1 && d.strategy == CAKE_RS_P2P_OWNER_PUSH;
  if (p2p && !plan->bound) return fail(CAKE_ERR_STATE, "cake_matmul_rs_bind_peers must be called before enqueue");
  if (!p2p && phases != (kPhasePush | kPhaseReduce))
    return fail(CAKE_ERR_STATE, "separate push / reduce phases exist only for the peer-to-peer strategy");
  if (p2p && !(phases & kPhasePush) && plan->epoch == 0)
    return fail(CAKE_ERR_STATE, "reduce phase enqueued before any push phase");
  int launches = 0;
  const size_t chunk_elems = static_cast<size_t>(plan->out_rows) * plan->out_cols;
  if (phases & kPhasePush) {
    const void* rhs_used = rhs;
    if (plan->rhs_via_transpose) {
      dim3 grid((d.n + 31) / 32, (d.k_local + 31) / 32), block(32, 8);
      cake::cake_transpose_bf16<<<grid, block, 0, stream>>>(static_cast<const uint16_t*>(rhs),
                                                            static_cast<uint16_t*>(plan->rhs_t),
                                                            (int)d.k_local, (int)d.n);
      CAKE_CUDA_TRY(cudaGetLastError());
      rhs_used = plan->rhs_t;
      ++launches;
    }
    if (lhs != plan->last_lhs || rhs_used != plan->last_rhs) {
      int32_t rc = encode_maps(plan, lhs, rhs_used);
      if (rc) return rc;
      plan->last_lhs = lhs;
      plan->last_rhs = rhs_used;
    }

    cake::MatmulParams p;
    memset(&p, 0, sizeof(p));
    p.m = (int)d.m;
    p.n = (int)d.n;
    p.k_local = (int)d.k_local;
    p.m_tiles = (int)((d.m + cake::kTileM - 1) / cake::kTileM);
    p.n_tiles = (int)((d.n + d.tile_n - 1) / d.tile_n);
    p.k_blocks = (int)((d.k_local + cake::kBlockK - 1) / cake::kBlockK);
    p.world = d.world;
    p.rank = d.rank;
    p.scatter_dim = d.scatter_dim;
    p.out_rows = (int)plan->out_rows;
    p.out_cols = (int)plan->out_cols;
    p.store_f32 = plan->tsize == 4;
    const int epp = 16 / (int)plan->tsize;
    p.vec_ok = (plan->out_cols % epp == 0) && (d.n % epp == 0);
    p.status = plan->status.dev;
    unsigned long long parity = 0;
    if (d.world == 1) {
      p.dest[0] = out;
    } else if (!p2p) {
      for (int o = 0; o < d.world; ++o) p.dest[o] = static_cast<char*>(out) + o * chunk_elems * plan->tsize;
    } else {
      plan->epoch += 1;
      parity = plan->epoch & 1ull;
      for (int o = 0; o < d.world; ++o) {
        p.dest[o] = static_cast<char*>(plan->slots[o]) + (parity * d.world + d.rank) * plan->slot_stride;
        p.flags_at[o] = static_cast<uint32_t*>(plan->flags[o]) + static_cast<size_t>(d.rank) * plan->quarters;
      }
      p.epoch = static_cast<uint32_t>(plan->epoch);
      p.quarters = plan->quarters;
      p.region_n_tiles = plan->region_n_tiles;
      p.push_done = plan->tickets + 2;
      if (phases & kPhaseReduce) {
        p.reduce_in_kernel = 1;
        fill_reduce_params(plan, parity, out, &p.red);
      }
    }
    // Tensor stores need 16-byte row pitch, and chunks (32 rows x 128 bytes) that never straddle owners.
    const int chunk_cols = 128 / (int)plan->tsize;
    const bool tma_ok = (plan->out_cols * plan->tsize) % 16 == 0 &&
                        (d.world == 1 || (d.scatter_dim == 0 ? plan->out_rows % 32 == 0 : plan->out_cols % chunk_cols == 0));
    const int maps_index = p2p ? (int)parity : 0;
    p.tma_store = tma_ok ? 1 : 0;
    if (tma_ok && plan->owner_maps_base[maps_index] != p.dest[0]) {
      for (int o = 0; o < d.world; ++o) {
        const uint64_t dims[2] = {static_cast<uint64_t>(plan->out_cols), static_cast<uint64_t>(plan->out_rows)};
        const uint64_t strides[1] = {static_cast<uint64_t>(plan->out_cols) * plan->tsize};
        const uint32_t box[2] = {static_cast<uint32_t>(chunk_cols), 32};
        int32_t mrc = cake::encode_tensor_map_typed(&plan->owner_maps[maps_index].m[o], p.dest[o], 2, dims, strides, box, true,
                                                    plan->tsize == 4 ? 4 : 2);
        if (mrc) return mrc;
      }
      plan->owner_maps_base[maps_index] = p.dest[0];
    }
    const int num_tiles = p.m_tiles * p.n_tiles;
    const int grid = num_tiles < plan->sm_count ? num_tiles : plan->sm_count;
    p.owner_rotation = 1;
    if (d.world > 1) {
      const bool aligned = d.scatter_dim == 0 ? (plan->out_rows % cake::kTileM == 0)
                                              : (plan->out_cols % d.tile_n == 0);
      p.region_order = aligned ? 1 : 0;
      // One wave of the grid covers grid / W tile groups: shift the owner sequence once per wave.
      p.owner_rotation = grid / d.world > 0 ? grid / d.world : 1;
      p.region_tiles = num_tiles / d.world;
      // How many of this rank's own tiles close the walk. With slack on the link, all of them: the
      // pushes then fall into the first (W - 1) / W of the contraction, which must still cover their
      // time on the link (estimated at 600 GB/s per GPU with every GPU pushing, against 1.6 PFLOP/s
      // of contraction). 8192 x 16384 x 8192 in bf16: on 2 and 4 GPUs yes (4 GPUs measured 0.432
      // against 0.445 ms with own tiles spread over the walk); at K / W = 2048 (8 GPUs, or K = 8192
      // on 4) the pushes need most of the link for the whole kernel and concentrating them costs
      // 2-12 %, also when only one or two waves of own tiles close the walk (K = 8192 on 4 GPUs:
      // 0.243 ms spread, 0.248 with a tail of two waves, 0.274 with all own tiles last).
      const double push_phase_s = (d.world - 1.0) / d.world * 2.0 * d.m * d.n * d.k_local / 1.6e15;
      const double link_s = (d.world - 1.0) / d.world * static_cast<double>(d.m) * d.n * plan->tsize / 600e9;
      p.own_tail = (p2p && p.region_order && link_s <= 0.8 * push_phase_s) ? p.region_tiles : 0;
      if (p2p) p.publish = (p.region_order && p.tma_store) ? cake::kPublishPerTile : cake::kPublishAtEnd;
      p.mailbox = (p.publish == cake::kPublishPerTile && p.quarters < (1 << 24)) ? 1 : 0;
      p.own_now = 1;  // 4 GPUs, 8192 x K x 8192: K = 16384 0.4356 -> 0.4306 ms, K = 12288 0.344 -> 0.339, K = 8192 unchanged
    }
    const bool kmajor = d.rhs_layout == 1 || plan->rhs_via_transpose;
    int32_t rc;
    if (d.tile_n == 256) rc = kmajor ? launch_gemm<256, true>(plan, p, grid, stream, maps_index) : launch_gemm<256, false>(plan, p, grid, stream, maps_index);
    else if (d.tile_n == 128) rc = kmajor ? launch_gemm<128, true>(plan, p, grid, stream, maps_index) : launch_gemm<128, false>(plan, p, grid, stream, maps_index);
    else rc = kmajor ? launch_gemm<64, true>(plan, p, grid, stream, maps_index) : launch_gemm<64, false>(plan, p, grid, stream, maps_index);
    if (rc) return rc;
    ++launches;
  } else if (p2p) {
    // The reduction of the most recent push, as a kernel of its own.
    cake::ReduceParams r;
    memset(&r, 0, sizeof(r));
    fill_reduce_params(plan, plan->epoch & 1ull, out, &r);
    const size_t chunks = (chunk_elems * plan->tsize + 4095) / 4096;
    int rgrid = (int)((chunks + 7) / 8);
    if (rgrid > plan->sm_count * 2) rgrid = plan->sm_count * 2;
    if (rgrid < 1) rgrid = 1;
    cake::cake_reduce_slots_sm100<<<rgrid, 256, 0, stream>>>(r);
    CAKE_CUDA_TRY(cudaGetLastError());
    ++launches;
  }
  plan->launches = launches;
  return CAKE_OK;
}
}  // namespace

extern "C" {

int32_t cake_matmul_rs_enqueue(cake_matmul_rs* plan, const void* lhs, const void* rhs, void* out,
                               void* stream) {
  return enqueue_impl(plan, lhs, rhs, out, stream, kPhasePush | kPhaseReduce);
}

int32_t cake_matmul_rs_enqueue_push(cake_matmul_rs* plan, const void* lhs, const void* rhs,
                                    void* stream) {
  // `out` is not written by the push phase of the peer-to-peer strategy; pass a non-null dummy.
  return enqueue_impl(plan, lhs, rhs, reinterpret_cast<void*>(16), stream, kPhasePush);
}

int32_t cake_matmul_rs_enqueue_reduce(cake_matmul_rs* plan, void* out, void* stream) {
  return enqueue_impl(plan, nullptr, nullptr, out, stream, kPhaseReduce);
}

}  // extern "C"

namespace {

// run_host at world 1 is bound by the host link: 2 (M + N) K bytes in, then the kernel, then M N
// elements out, one after the other. The rows of lhs are independent, so the matrix is cut into
// blocks of rows: once rhs is on the device, block i is contracted while block i + 1 arrives and
// block i - 1 leaves (the link carries both directions at once). Every output element is still
// accumulated over K in the same order, so the result does not depend on the cut. The cut is used
// when the blocks are whole tiles and at least 8 MiB of lhs each.
int32_t prepare_row_blocks(cake_matmul_rs* plan) {
  if (plan->host_blocks != 0) return CAKE_OK;
  const cake_matmul_rs_desc& d = plan->d;
  plan->host_blocks = 1;
  if (plan->rhs_via_transpose) return CAKE_OK;
  int blocks = 0;
  for (int candidate = cake_matmul_rs::kHostBlocks; candidate >= 2; candidate /= 2) {
    const int64_t rows = d.m / candidate;
    if (d.m % candidate == 0 && rows % cake::kTileM == 0 && rows * d.k_local * 2 >= (8ll << 20)) {
      blocks = candidate;
      break;
    }
  }
  if (blocks == 0) return CAKE_OK;
  cake_matmul_rs_desc block_desc = d;
  block_desc.m = d.m / blocks;
  int32_t rc = cake_matmul_rs_create(&block_desc, &plan->row_block_plan);
  if (rc) return rc;
  CAKE_CUDA_TRY(cudaStreamCreateWithFlags(&plan->copy_in, cudaStreamNonBlocking));
  CAKE_CUDA_TRY(cudaStreamCreateWithFlags(&plan->copy_out, cudaStreamNonBlocking));
  CAKE_CUDA_TRY(cudaEventCreateWithFlags(&plan->host_begin, cudaEventDisableTiming));
  CAKE_CUDA_TRY(cudaEventCreateWithFlags(&plan->host_end, cudaEventDisableTiming));
  for (int i = 0; i < blocks; ++i) {
    CAKE_CUDA_TRY(cudaEventCreateWithFlags(&plan->block_in[i], cudaEventDisableTiming));
    CAKE_CUDA_TRY(cudaEventCreateWithFlags(&plan->block_done[i], cudaEventDisableTiming));
  }
  plan->host_blocks = blocks;
  return CAKE_OK;
}

int32_t run_host_row_blocks(cake_matmul_rs* plan, const void* lhs_host, const void* rhs_host, void* out_host,
                            cudaStream_t stream) {
  const cake_matmul_rs_desc& d = plan->d;
  const int blocks = plan->host_blocks;
  const size_t lhs_block = static_cast<size_t>(d.m / blocks) * d.k_local * 2;
  const size_t out_block = static_cast<size_t>(d.m / blocks) * d.n * plan->osize;
  const size_t rhs_bytes = static_cast<size_t>(d.n) * d.k_local * 2;
  // The copies start after whatever the caller has already queued on its stream.
  CAKE_CUDA_TRY(cudaEventRecord(plan->host_begin, stream));
  CAKE_CUDA_TRY(cudaStreamWaitEvent(plan->copy_in, plan->host_begin, 0));
  CAKE_CUDA_TRY(cudaStreamWaitEvent(plan->copy_out, plan->host_begin, 0));
  CAKE_CUDA_TRY(cudaMemcpyAsync(plan->h_rhs, rhs_host, rhs_bytes, cudaMemcpyHostToDevice, plan->copy_in));
  for (int i = 0; i < blocks; ++i) {
    CAKE_CUDA_TRY(cudaMemcpyAsync(static_cast<char*>(plan->h_lhs) + i * lhs_block, static_cast<const char*>(lhs_host) + i * lhs_block,
                                  lhs_block, cudaMemcpyHostToDevice, plan->copy_in));
    CAKE_CUDA_TRY(cudaEventRecord(plan->block_in[i], plan->copy_in));
  }
  for (int i = 0; i < blocks; ++i) {
    CAKE_CUDA_TRY(cudaStreamWaitEvent(stream, plan->block_in[i], 0));
    int32_t rc = cake_matmul_rs_enqueue(plan->row_block_plan, static_cast<char*>(plan->h_lhs) + i * lhs_block, plan->h_rhs,
                                        static_cast<char*>(plan->h_out) + i * out_block, stream);
    if (rc) return rc;
    CAKE_CUDA_TRY(cudaEventRecord(plan->block_done[i], stream));
    CAKE_CUDA_TRY(cudaStreamWaitEvent(plan->copy_out, plan->block_done[i], 0));
    CAKE_CUDA_TRY(cudaMemcpyAsync(static_cast<char*>(out_host) + i * out_block, static_cast<char*>(plan->h_out) + i * out_block,
                                  out_block, cudaMemcpyDeviceToHost, plan->copy_out));
  }
  CAKE_CUDA_TRY(cudaEventRecord(plan->host_end, plan->copy_out));
  CAKE_CUDA_TRY(cudaStreamWaitEvent(stream, plan->host_end, 0));
  CAKE_CUDA_TRY(cudaStreamSynchronize(stream));
  // A barrier of a row block's kernel that gave up is reported like one of the whole matrix's.
  cake_status block_status;
  return cake_matmul_rs_status(plan->row_block_plan, stream, &block_status);
}

}  // namespace

extern "C" {

int32_t cake_matmul_rs_run_host(cake_matmul_rs* plan, const void* lhs_host, const void* rhs_host,
                                void* out_host, void* stream_v) {
  if (!plan || !lhs_host || !rhs_host || !out_host) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_matmul_rs_run_host: null argument");
  const cake_matmul_rs_desc& d = plan->d;
  if (d.world > 1 && d.strategy != CAKE_RS_P2P_OWNER_PUSH)
    return fail(CAKE_ERR_UNSUPPORTED, "run_host needs world == 1 or the peer-to-peer strategy");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const size_t lhs_bytes = static_cast<size_t>(d.m) * d.k_local * 2;
  const size_t rhs_bytes = static_cast<size_t>(d.n) * d.k_local * 2;
  const size_t out_bytes = static_cast<size_t>(plan->out_rows) * plan->out_cols * plan->osize;
  if (!plan->h_lhs) CAKE_CUDA_TRY(cudaMalloc(&plan->h_lhs, lhs_bytes));
  if (!plan->h_rhs) CAKE_CUDA_TRY(cudaMalloc(&plan->h_rhs, rhs_bytes));
  if (!plan->h_out) CAKE_CUDA_TRY(cudaMalloc(&plan->h_out, out_bytes));
  if (d.world == 1) {
    int32_t prc = prepare_row_blocks(plan);
    if (prc) return prc;
    if (plan->host_blocks > 1) return run_host_row_blocks(plan, lhs_host, rhs_host, out_host, stream);
  }
  CAKE_CUDA_TRY(cudaMemcpyAsync(plan->h_lhs, lhs_host, lhs_bytes, cudaMemcpyHostToDevice, stream));
  CAKE_CUDA_TRY(cudaMemcpyAsync(plan->h_rhs, rhs_host, rhs_bytes, cudaMemcpyHostToDevice, stream));
  int32_t rc = cake_matmul_rs_enqueue(plan, plan->h_lhs, plan->h_rhs, plan->h_out, stream_v);
  if (rc) return rc;
  CAKE_CUDA_TRY(cudaMemcpyAsync(out_host, plan->h_out, out_bytes, cudaMemcpyDeviceToHost, stream));
  CAKE_CUDA_TRY(cudaStreamSynchronize(stream));
  return CAKE_OK;
}

int32_t cake_matmul_rs_status(cake_matmul_rs* plan, void* stream_v, cake_status* out) {
  if (!plan || !out) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_matmul_rs_status: null argument");
  int32_t rc = plan->status.read_and_clear(static_cast<cudaStream_t>(stream_v), out);
  if (rc) return rc;
  if (out->code == 1 || out->code == 2)
    return fail(CAKE_ERR_TIMEOUT, "device-side bounded wait ran out: code=%d block=%d tile/src=%d where=%d",
                out->code, out->detail0, out->detail1, out->detail2);
  return CAKE_OK;
}

}  // extern "C"
