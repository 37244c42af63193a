// Ragged paged attention, pure decode, for sm_100a (HBM-bound).
//
// What it replaces: the per-sequence loop of _owned_rpa_kernel_loop
// (src/tpu_cake/rpa_owned_kernel.py:85-960; page fetch _fetch_bkv :417-471, online softmax
// :199-358) and the executor FusedRpaPlan.invoke hands its inputs to
// (src/tpu_cake/rpa_lowering.py:232-273). Arithmetic follows the reference oracles
// inkling_rpa_reference (src/tpu_cake/workloads/inkling_rpa.py:37-73) and
// inkling_fused_rpa_reference (:471-589).
//
// Kernels
//   cake_rpa_plan_sm100      one CTA: per-sequence chunk counts -> exclusive prefix (work-item
//                            table), reset of the work counter and of the arrival counters
//   cake_rpa_cache_update_sm100  optional: writes each sequence's new K/V at position kv_len-1
//   cake_rpa_decode_sm100    persistent; every WARP is an independent worker with its own
//                            3-stage shared-memory ring. A work item is (sequence, KV head,
//                            chunk of the KV range). Pages are gathered through the page table
//                            with one TMA box per page (128-byte swizzle, never multicast); all
//                            query heads of the KV head share the page (GQA: each page is read
//                            once per KV head). QK^T and PV run on mma.sync m16n8k16 with the
//                            query-head group padded to 16 rows; online softmax in f32 with
//                            quad shuffles.
//                            Split-KV partials (m, l, o) of a (sequence, KV head) are merged, in
//                            chunk order, by whichever warp publishes the last chunk; loads run
//                            ahead into the next work item so the ring never drains.
#include <cuda_bf16.h>
#include <math.h>
#include <string.h>

#include <new>

#include "cake_host.h"
#include "cake_ptx.cuh"

namespace cake {

#ifndef CAKE_RPA_WARPS
#define CAKE_RPA_WARPS 6
#endif
#ifndef CAKE_RPA_STAGES
#define CAKE_RPA_STAGES 2
#endif
constexpr int kRpaWarps = CAKE_RPA_WARPS;
constexpr int kRpaThreads = kRpaWarps * 32;
constexpr int kRpaStages = CAKE_RPA_STAGES;
constexpr int kStageTokens = 32;
constexpr int kRowBytes = 256;                                // one token of one head: 128 bf16
constexpr int kStageBytes = kStageTokens * 2 * kRowBytes;     // K and V: 16 KiB
constexpr int kRpaSmemBytes = kRpaWarps * kRpaStages * kStageBytes + 1024 + 256;
constexpr long long kRpaBarrierBudget = 2000000000ll;
constexpr float kNegBig = -1.0e30f;

struct RpaParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int32_t* kv_lens;
  const int32_t* page_table;
  const int32_t* cu_kv_lens;
  int32_t num_seqs, q_heads, kv_heads, group, head_dim;
  int32_t page_size, log2_ps;
  int32_t table_layout, max_pages_per_seq, table_len;
  int32_t total_pages;
  int32_t fused;
  int32_t chunk_tokens;
  float scale_log2;  // sm_scale * log2(e)
  int32_t bias_mode;
  const float* bias;  // mode 1: [q_heads, bias_extent]
  int32_t bias_extent;
  const __nv_bfloat16* rel_states;  // mode 2: [num_seqs, q_heads, rel_dim]
  const __nv_bfloat16* rel_proj;    // mode 2: [rel_dim, bias_extent]
  int32_t rel_dim;
  int32_t* work_counter;
  int32_t* arrive;     // [num_seqs * kv_heads] chunks published per (sequence, KV head)
  int32_t* item_base;  // [num_seqs + 1] exclusive prefix of per-sequence chunk counts
  int32_t* item_seq;   // [sum of chunk counts] sequence of every (sequence, chunk) pair
  float* part_o;       // [max_items][group][128]
  float* part_ml;      // [max_items][group][2]
  int32_t max_items;
  int32_t* status;
};

__device__ __forceinline__ void rpa_record(int32_t* status, int code, int d0, int d1, int d2) {
  if (status && atomicCAS(status, 0, code) == 0) {
    status[1] = d0;
    status[2] = d1;
    status[3] = d2;
  }
}

__global__ void __launch_bounds__(256) cake_rpa_plan_sm100(RpaParams p) {
  __shared__ int s_scan[256];
  __shared__ int s_carry;
  if (threadIdx.x == 0) {
    s_carry = 0;
    *p.work_counter = 0;
    p.item_base[0] = 0;
  }
  for (int i = threadIdx.x; i < p.num_seqs * p.kv_heads; i += blockDim.x) p.arrive[i] = 0;
  __syncthreads();
  for (int base = 0; base < p.num_seqs; base += 256) {
    const int s = base + threadIdx.x;
    int chunks = 0;
    if (s < p.num_seqs) {
      const int len = p.kv_lens[s];
      if (len > 0) chunks = (len + p.chunk_tokens - 1) / p.chunk_tokens;
      if (len < 0) rpa_record(p.status, 4, s, len, 0);
    }
    s_scan[threadIdx.x] = chunks;
    __syncthreads();
    for (int off = 1; off < 256; off <<= 1) {
      int v = 0;
      if (threadIdx.x >= off) v = s_scan[threadIdx.x - off];
      __syncthreads();
      s_scan[threadIdx.x] += v;
      __syncthreads();
    }
    if (s < p.num_seqs) {
      const int end = s_carry + s_scan[threadIdx.x];
      p.item_base[s + 1] = end;
      if (static_cast<long long>(end) * p.kv_heads <= p.max_items)
        for (int c = end - chunks; c < end; ++c) p.item_seq[c] = s;
    }
    __syncthreads();
    if (threadIdx.x == 255) s_carry += s_scan[255];
    __syncthreads();
  }
}

// Logical page slot -> physical page for token `tok` of sequence `s`.
__device__ __forceinline__ int rpa_page_lookup(const RpaParams& p, int s, int page_slot) {
  if (p.table_layout == CAKE_RPA_TABLE_2D) {
    return p.page_table[static_cast<size_t>(s) * p.max_pages_per_seq + page_slot];
  }
  const int idx = (p.cu_kv_lens[s] >> p.log2_ps) + page_slot;
  if (idx < 0 || idx >= p.table_len) return -1;
  return p.page_table[idx];
}

// Writes new_k/new_v [num_seqs, kv_heads, head_dim] at position kv_len-1 of each sequence.
// Fused cache rows are zero-filled beyond head_dim up to the padded width, as the reference
// oracle does (src/tpu_cake/workloads/inkling_rpa.py:518-534).
__global__ void cake_rpa_cache_update_sm100(RpaParams p, const __nv_bfloat16* new_k,
                                            const __nv_bfloat16* new_v, __nv_bfloat16* cache0,
                                            __nv_bfloat16* cache1) {
  const int s = blockIdx.x;
  const int len = p.kv_lens[s];
  if (len <= 0) return;
  const int pos = len - 1;
  const int page = rpa_page_lookup(p, s, pos >> p.log2_ps);
  if (page < 0 || page >= p.total_pages) {
    if (threadIdx.x == 0) rpa_record(p.status, 3, s, pos >> p.log2_ps, page);
    return;
  }
  const int slot = pos & (p.page_size - 1);
  for (int i = threadIdx.x; i < p.kv_heads * 2 * 128; i += blockDim.x) {
    const int d = i & 127;
    const int kv = (i >> 7) & 1;
    const int h = i >> 8;
    const __nv_bfloat16* src = kv ? new_v : new_k;
    const __nv_bfloat16 val = d < p.head_dim
                                  ? src[(static_cast<size_t>(s) * p.kv_heads + h) * p.head_dim + d]
                                  : __float2bfloat16_rn(0.f);
    if (p.fused) {
      const size_t row = (static_cast<size_t>(page) * p.page_size + slot) * (2 * p.kv_heads) + 2 * h + kv;
      cache0[row * 128 + d] = val;
    } else if (d < p.head_dim) {
      __nv_bfloat16* dst = kv ? cache1 : cache0;
      dst[((static_cast<size_t>(page) * p.page_size + slot) * p.kv_heads + h) * 128 + d] = val;
    }
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                            uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                                  uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// Byte offset inside a stage of the 16-byte chunk `c16` (0..15) of token `t`'s K (kv=0) or V
// (kv=1) row, including the 128-byte swizzle the TMA applied (address bits [7,10) xor into
// [4,7); the stage base is 1024-byte aligned).
__device__ __forceinline__ uint32_t rpa_smem_off(int t, int c16, int kv, int page_size, int log2_ps) {
  const int pg = t >> log2_ps;
  const int tp = t & (page_size - 1);
  uint32_t off = static_cast<uint32_t>(pg * page_size * 512 + kv * page_size * 256 +
                                       (c16 >> 3) * page_size * 128 + tp * 128 + (c16 & 7) * 16);
  return off ^ (((off >> 7) & 7u) << 4);
}

// One unit of work of a warp: KV tokens [tok0, tok0 + ntok) of one (sequence, KV head).
struct RpaItem {
  int id, s, h, n_chunks, len, tok0;
};

// Claims the next work item from the global queue and decodes it (warp-uniform). Returns false
// when the queue is exhausted.
__device__ __forceinline__ bool rpa_fetch_item(const RpaParams& p, int total_items, int lane,
                                               RpaItem& it) {
  int id = 0;
  if (lane == 0) id = atomicAdd(p.work_counter, 1);
  id = __shfl_sync(0xffffffffu, id, 0);
  if (id >= total_items) return false;
  if (id >= p.max_items) {
    if (lane == 0) rpa_record(p.status, 4, id, p.max_items, 1);
    return false;
  }
  const int cs = id / p.kv_heads;
  const int lo = p.item_seq[cs];
  const int base = p.item_base[lo];
  it.id = id;
  it.s = lo;
  it.h = id - cs * p.kv_heads;
  it.n_chunks = p.item_base[lo + 1] - base;
  it.len = p.kv_lens[lo];
  it.tok0 = (cs - base) * p.chunk_tokens;
  return true;
}

__device__ __forceinline__ int rpa_item_tokens(const RpaParams& p, const RpaItem& it) {
  return min(p.chunk_tokens, it.len - it.tok0);
}

// Issues the TMA loads of stage `st` of item `it` into the ring slot at `stage_smem`: one box per
// page (K and V of one KV head). Page ids are read from the page table 32 at a time (one per
// lane, `window_pages`, for the item-relative page window `window`) and handed to the issuing
// lanes by shuffle, so a stage does not wait on a table read of its own.
__device__ __forceinline__ void rpa_issue_stage(const RpaParams& p, const CUtensorMap* tmap_k,
                                                const CUtensorMap* tmap_v, const RpaItem& it, int st,
                                                uint32_t stage_smem, uint32_t bar, int lane,
                                                int& window, int& window_pages) {
  const int ps = p.page_size;
  const int pages_per_stage = kStageTokens >> p.log2_ps;
  const int ntok = rpa_item_tokens(p, it);
  const int rem = ntok - st * kStageTokens;
  const int npages = min(pages_per_stage, (rem + ps - 1) >> p.log2_ps);
  const int first = st * pages_per_stage;  // first page of the stage, relative to the item
  if ((first >> 5) != window) {
    window = first >> 5;
    const int rel = window * 32 + lane;
    int page = p.total_pages;  // an out-of-bounds coordinate: the TMA unit fills the box with zeros
    if (rel < ((ntok + ps - 1) >> p.log2_ps)) {
      const int page_slot = (it.tok0 >> p.log2_ps) + rel;
      page = rpa_page_lookup(p, it.s, page_slot);
      if (page < 0 || page >= p.total_pages) {
        rpa_record(p.status, 3, it.s, page_slot, page);
        page = p.total_pages;
      }
    }
    window_pages = page;
  }
  const int page = __shfl_sync(0xffffffffu, window_pages, (first + lane) & 31);
  if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(npages * ps * 512));
  __syncwarp();
  if (lane < npages) {
    const uint32_t dst = stage_smem + lane * ps * 512;
    if (p.fused) {
      tma_load_5d(dst, tmap_k, bar, 0, 0, 0, 2 * it.h, page);
    } else {
      tma_load_5d(dst, tmap_k, bar, 0, 0, 0, it.h, page);
      tma_load_5d(dst + ps * 256, tmap_v, bar, 0, 0, 0, it.h, page);
    }
  }
}

__global__ void __launch_bounds__(kRpaThreads, 1)
    cake_rpa_decode_sm100(const __grid_constant__ CUtensorMap tmap_k,
                          const __grid_constant__ CUtensorMap tmap_v, const RpaParams p) {
  extern __shared__ uint8_t rpa_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(rpa_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  uint8_t* ring = smem + warp * kRpaStages * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kRpaWarps * kRpaStages * kStageBytes) +
                   warp * kRpaStages;
  if (lane == 0) {
    for (int s = 0; s < kRpaStages; ++s) mbar_init(smem_u32(&bars[s]), 1);
    fence_mbar_init();
    if (warp == 0) {
      prefetch_tensormap(&tmap_k);
      prefetch_tensormap(&tmap_v);
    }
  }
  __syncwarp();

  const int ps = p.page_size;
  const int total_items = p.item_base[p.num_seqs] * p.kv_heads;
  const int row0 = lane >> 2;
  const int row1 = row0 + 8;
  const int quad = lane & 3;

  // The warp streams stages through its ring continuously: `consume_pos` counts stages computed,
  // `issue_pos` stages whose loads were issued; loads run ahead across the boundary into the next
  // work item so the ring never drains between items.
  RpaItem cur, nxt;
  bool nxt_fetched = false, have_nxt = false;
  int cur_issued = 0, nxt_issued = 0;
  int cur_window = -1, nxt_window = -1, cur_pages = 0, nxt_pages = 0;
  uint32_t issue_pos = 0, consume_pos = 0;
  bool alive = rpa_fetch_item(p, total_items, lane, cur);

  while (alive) {
    const int h = cur.h, s = cur.s, len = cur.len, tok0 = cur.tok0;
    const int ntok = rpa_item_tokens(p, cur);
    const int nstages = (ntok + kStageTokens - 1) / kStageTokens;

    // ---- query fragments (A operand, 16 x 128, rows >= group are zero)
    uint32_t qa[8][4];
    {
      const size_t qrow0 = (static_cast<size_t>(s) * p.q_heads + h * p.group + row0) * p.head_dim;
      const size_t qrow1 = (static_cast<size_t>(s) * p.q_heads + h * p.group + row1) * p.head_dim;
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        const int k = ks * 16 + quad * 2;
        qa[ks][0] = (row0 < p.group && k < p.head_dim) ? *reinterpret_cast<const uint32_t*>(p.q + qrow0 + k) : 0u;
        qa[ks][1] = (row1 < p.group && k < p.head_dim) ? *reinterpret_cast<const uint32_t*>(p.q + qrow1 + k) : 0u;
        qa[ks][2] = (row0 < p.group && k + 8 < p.head_dim) ? *reinterpret_cast<const uint32_t*>(p.q + qrow0 + k + 8) : 0u;
        qa[ks][3] = (row1 < p.group && k + 8 < p.head_dim) ? *reinterpret_cast<const uint32_t*>(p.q + qrow1 + k + 8) : 0u;
      }
    }

    float oacc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    float m_run[2] = {kNegBig, kNegBig};
    float l_run[2] = {0.f, 0.f};

    for (int st = 0; st < nstages; ++st) {
      // ---- top up the ring. A slot is refilled only after every lane finished reading it
      // (__syncwarp at the end of the previous stage) and a proxy fence orders those generic-proxy
      // reads before the async-proxy writes of the new TMA.
      fence_proxy_async_smem();
      auto top_up = [&]() {
      while (issue_pos - consume_pos < static_cast<uint32_t>(kRpaStages)) {
        const uint32_t slot = issue_pos % kRpaStages;
        const uint32_t stage_smem = smem_u32(ring + slot * kStageBytes);
        const uint32_t bar = smem_u32(&bars[slot]);
        if (cur_issued < nstages) {
          rpa_issue_stage(p, &tmap_k, &tmap_v, cur, cur_issued, stage_smem, bar, lane, cur_window, cur_pages);
          ++cur_issued;
          ++issue_pos;
          continue;
        }
        if (!nxt_fetched || !have_nxt) break;
        const int nxt_stages = (rpa_item_tokens(p, nxt) + kStageTokens - 1) / kStageTokens;
        if (nxt_issued >= nxt_stages) break;
        rpa_issue_stage(p, &tmap_k, &tmap_v, nxt, nxt_issued, stage_smem, bar, lane, nxt_window, nxt_pages);
        ++nxt_issued;
        ++issue_pos;
      }
      };
      top_up();
      if (!nxt_fetched) {
        // Claim the next item now: its queue and table reads overlap the wait for this stage's
        // data, and the ring can then run ahead into it without stalling.
        nxt_fetched = true;
        nxt_issued = 0;
        nxt_window = -1;
        have_nxt = rpa_fetch_item(p, total_items, lane, nxt);
        if (have_nxt && lane < 2 * p.group) {
          // Pull the next item's query rows toward L2 so its fragment loads do not stall.
          const char* qptr = reinterpret_cast<const char*>(
              p.q + (static_cast<size_t>(nxt.s) * p.q_heads + nxt.h * p.group + (lane >> 1)) * p.head_dim);
          if ((lane & 1) * 128 < p.head_dim * 2)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(qptr + (lane & 1) * 128));
        }
        top_up();  // a short item may leave room to run ahead into the one just claimed
      }
      const uint32_t slot = consume_pos % kRpaStages;
      const uint32_t parity = (consume_pos / kRpaStages) & 1u;
      const bool arrived = mbar_wait_bounded(smem_u32(&bars[slot]), parity, kRpaBarrierBudget);
      if (!__all_sync(0xffffffffu, arrived)) {
        if (lane == 0) rpa_record(p.status, 1, blockIdx.x, cur.id, st);
        alive = false;
        break;
      }
      const uint32_t sbase = smem_u32(ring + slot * kStageBytes);
      const int valid = min(kStageTokens, ntok - st * kStageTokens);
      const int n16 = (valid + 15) >> 4;  // 16-token groups to process (1 or 2)

      // Zero V rows between the last valid token and the end of its 16-token group: their
      // contents are stale or uninitialised and 0 * NaN would poison the accumulator.
      if (valid < n16 * 16) {
        for (int t = valid; t < n16 * 16; ++t) {
          if (lane < 16) {
            const uint32_t off = rpa_smem_off(t, lane, 1, ps, p.log2_ps);
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(sbase + off), "r"(0u) : "memory");
          }
        }
        __syncwarp();
      }

      // ---- S = Q K^T for up to 32 tokens
      float sacc[4][4];
#pragma unroll
      for (int j = 0; j < 4; ++j) sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f;
#pragma unroll
      for (int g16 = 0; g16 < 2; ++g16) {
        if (g16 < n16) {
          const int t = g16 * 16 + (lane & 7) + ((lane >> 4) << 3);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            uint32_t b0, b1, b2, b3;
            ldmatrix_x4(sbase + rpa_smem_off(t, ks * 2 + ((lane >> 3) & 1), 0, ps, p.log2_ps), b0, b1, b2, b3);
            mma_bf16_16816(sacc[g16 * 2], qa[ks], b0, b1);
            mma_bf16_16816(sacc[g16 * 2 + 1], qa[ks], b2, b3);
          }
        }
      }

      // ---- scale, bias, mask, online softmax (rows row0 and row1 of this thread)
      const int pos_base = tok0 + st * kStageTokens;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tk = j * 8 + quad * 2 + (e & 1);
          const int row = (e < 2) ? row0 : row1;
          float v = sacc[j][e] * p.scale_log2;
          const int pos = pos_base + tk;
          if (p.bias_mode != 0 && row < p.group && tk < valid) {
            const int head = h * p.group + row;
            float b = 0.f;
            if (p.bias_mode == 1) {
              if (pos < p.bias_extent) b = p.bias[static_cast<size_t>(head) * p.bias_extent + pos];
            } else {
              const int dist = len - 1 - pos;
              if (dist < p.bias_extent) {
                const __nv_bfloat16* st_row = p.rel_states + (static_cast<size_t>(s) * p.q_heads + head) * p.rel_dim;
                for (int r = 0; r < p.rel_dim; ++r)
                  b += __bfloat162float(st_row[r]) *
                       __bfloat162float(p.rel_proj[static_cast<size_t>(r) * p.bias_extent + dist]);
              }
            }
            v += b * 1.4426950408889634f;
          }
          sacc[j][e] = (tk < valid) ? v : kNegBig;
        }
      }
      float mx0 = kNegBig, mx1 = kNegBig;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mx0 = fmaxf(mx0, fmaxf(sacc[j][0], sacc[j][1]));
        mx1 = fmaxf(mx1, fmaxf(sacc[j][2], sacc[j][3]));
      }
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
      const float al0 = exp2f(m_run[0] - mn0), al1 = exp2f(m_run[1] - mn1);
      m_run[0] = mn0;
      m_run[1] = mn1;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        sacc[j][0] = exp2f(sacc[j][0] - mn0);
        sacc[j][1] = exp2f(sacc[j][1] - mn0);
        sacc[j][2] = exp2f(sacc[j][2] - mn1);
        sacc[j][3] = exp2f(sacc[j][3] - mn1);
        sum0 += sacc[j][0] + sacc[j][1];
        sum1 += sacc[j][2] + sacc[j][3];
      }
      l_run[0] = l_run[0] * al0 + sum0;
      l_run[1] = l_run[1] * al1 + sum1;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        oacc[i][0] *= al0;
        oacc[i][1] *= al0;
        oacc[i][2] *= al1;
        oacc[i][3] *= al1;
      }

      // ---- O += P V
#pragma unroll
      for (int g16 = 0; g16 < 2; ++g16) {
        if (g16 < n16) {
          uint32_t pa[4];
          pa[0] = pack_bf16(sacc[g16 * 2][0], sacc[g16 * 2][1]);
          pa[1] = pack_bf16(sacc[g16 * 2][2], sacc[g16 * 2][3]);
          pa[2] = pack_bf16(sacc[g16 * 2 + 1][0], sacc[g16 * 2 + 1][1]);
          pa[3] = pack_bf16(sacc[g16 * 2 + 1][2], sacc[g16 * 2 + 1][3]);
          const int t = g16 * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
          for (int nd = 0; nd < 8; ++nd) {
            uint32_t v0, v1, v2, v3;
            ldmatrix_x4_trans(sbase + rpa_smem_off(t, nd * 2 + (lane >> 4), 1, ps, p.log2_ps), v0, v1, v2, v3);
            mma_bf16_16816(oacc[nd * 2], pa, v0, v1);
            mma_bf16_16816(oacc[nd * 2 + 1], pa, v2, v3);
          }
        }
      }
      __syncwarp();
      ++consume_pos;
    }
    if (!alive) break;

    // ---- finish the item: row sums across the quad, then output or partial
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 1);
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], 2);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 1);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], 2);
    if (cur.n_chunks == 1) {
      const float inv0 = 1.f / l_run[0], inv1 = 1.f / l_run[1];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int d = i * 8 + quad * 2;
        if (d < p.head_dim) {
          if (row0 < p.group)
            *reinterpret_cast<uint32_t*>(p.out + (static_cast<size_t>(s) * p.q_heads + h * p.group + row0) * p.head_dim + d) =
                pack_bf16(oacc[i][0] * inv0, oacc[i][1] * inv0);
          if (row1 < p.group)
            *reinterpret_cast<uint32_t*>(p.out + (static_cast<size_t>(s) * p.q_heads + h * p.group + row1) * p.head_dim + d) =
                pack_bf16(oacc[i][2] * inv1, oacc[i][3] * inv1);
        }
      }
    } else {
      float* po = p.part_o + static_cast<size_t>(cur.id) * p.group * 128;
      float* pml = p.part_ml + static_cast<size_t>(cur.id) * p.group * 2;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int d = i * 8 + quad * 2;
        if (row0 < p.group) *reinterpret_cast<float2*>(po + row0 * 128 + d) = make_float2(oacc[i][0], oacc[i][1]);
        if (row1 < p.group) *reinterpret_cast<float2*>(po + row1 * 128 + d) = make_float2(oacc[i][2], oacc[i][3]);
      }
      if (quad == 0) {
        if (row0 < p.group) *reinterpret_cast<float2*>(pml + row0 * 2) = make_float2(m_run[0], l_run[0]);
        if (row1 < p.group) *reinterpret_cast<float2*>(pml + row1 * 2) = make_float2(m_run[1], l_run[1]);
      }
      // Publish the partial; the warp that publishes the last chunk of this (sequence, KV head)
      // merges all of them, always in chunk order, so the result does not depend on who merges.
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        __threadfence();  // cumulative over the other lanes' stores, ordered before it by the warp sync
        last = atomicAdd(p.arrive + s * p.kv_heads + h, 1) == cur.n_chunks - 1;
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
        __threadfence();
        const size_t first_item = static_cast<size_t>(cur.id / p.kv_heads - tok0 / p.chunk_tokens) * p.kv_heads + h;
        const int n = cur.n_chunks;
        for (int r = 0; r < p.group; ++r) {
          // Lane c reads chunk c's (m, l); the running maximum and the sum come from shuffles.
          float m = kNegBig;
          for (int c0 = 0; c0 < n; c0 += 32) {
            const int c = c0 + lane;
            if (c < n) m = fmaxf(m, __ldcg(p.part_ml + ((first_item + static_cast<size_t>(c) * p.kv_heads) * p.group + r) * 2));
          }
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
          float l = 0.f;
          float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int c0 = 0; c0 < n; c0 += 32) {
            const int c = c0 + lane;
            float w = 0.f;
            if (c < n) {
              const float2 ml = __ldcg(reinterpret_cast<const float2*>(
                  p.part_ml + ((first_item + static_cast<size_t>(c) * p.kv_heads) * p.group + r) * 2));
              w = exp2f(ml.x - m);
              l += ml.y * w;
            }
            const int cnt = min(32, n - c0);
#pragma unroll 4
            for (int jj = 0; jj < cnt; ++jj) {  // fixed chunk order; independent loads pipeline
              const float wj = __shfl_sync(0xffffffffu, w, jj);
              const size_t row = (first_item + static_cast<size_t>(c0 + jj) * p.kv_heads) * p.group + r;
              const float4 v = __ldcg(reinterpret_cast<const float4*>(p.part_o + row * 128) + lane);
              o.x += v.x * wj;
              o.y += v.y * wj;
              o.z += v.z * wj;
              o.w += v.w * wj;
            }
          }
#pragma unroll
          for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
          const float inv = 1.f / l;
          if (lane * 4 < p.head_dim) {
            uint2 packed;
            packed.x = pack_bf16(o.x * inv, o.y * inv);
            packed.y = pack_bf16(o.z * inv, o.w * inv);
            *reinterpret_cast<uint2*>(p.out + (static_cast<size_t>(s) * p.q_heads + h * p.group + r) * p.head_dim + lane * 4) = packed;
          }
        }
      }
    }

    // ---- next item (already claimed and partly in flight if the ring ran ahead)
    if (!nxt_fetched) {
      nxt_issued = 0;
      nxt_window = -1;
      have_nxt = rpa_fetch_item(p, total_items, lane, nxt);
    }
    if (!have_nxt) break;
    cur = nxt;
    cur_issued = nxt_issued;
    cur_window = nxt_window;
    cur_pages = nxt_pages;
    nxt_fetched = false;
    have_nxt = false;
  }

  if (!alive) {
    // A wait ran out: let loads already issued land before shared memory is released.
    for (uint32_t pos = consume_pos; pos < issue_pos; ++pos)
      mbar_wait_bounded(smem_u32(&bars[pos % kRpaStages]), (pos / kRpaStages) & 1u, 100000000ll);
  }
}

}  // namespace cake

// ====================================================================================== host

struct cake_rpa {
  cake_rpa_desc d;
  int sm_count = 0;
  int log2_ps = 0;
  int chunk_tokens = 0;
  int64_t max_items = 0;
  size_t off_item_base = 0, off_item_seq = 0, off_arrive = 0, off_part_o = 0, off_part_ml = 0, ws_bytes = 0;
  cake::StatusWord status;
  const void* last_c0 = nullptr;
  const void* last_c1 = nullptr;
  CUtensorMap tmap_k, tmap_v;
  int launches = 0;
};

namespace {
using cake::fail;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Workspace: [work counter | item_base | item_seq | arrival counters | partial (m,l) | partial o].
void rpa_layout_workspace(cake_rpa* plan, int group) {
  const cake_rpa_desc& d = plan->d;
  plan->off_item_base = 256;
  plan->off_item_seq = align_up(plan->off_item_base + sizeof(int32_t) * (d.num_seqs + 1), 256);
  plan->off_arrive = align_up(plan->off_item_seq + sizeof(int32_t) * (plan->max_items / d.kv_heads + 1), 256);
  plan->off_part_ml = align_up(plan->off_arrive + sizeof(int32_t) * d.num_seqs * d.kv_heads, 256);
  plan->off_part_o = align_up(plan->off_part_ml + sizeof(float) * 2 * group * plan->max_items, 256);
  plan->ws_bytes = plan->off_part_o + sizeof(float) * 128 * group * plan->max_items;
}

int32_t rpa_encode_maps(cake_rpa* plan, const void* c0, const void* c1) {
  const cake_rpa_desc& d = plan->d;
  const uint64_t ps = d.page_size;
  if (d.cache_layout == CAKE_RPA_CACHE_FUSED) {
    const uint64_t heads2 = 2ull * d.kv_heads;
    const uint64_t dims[5] = {64, ps, 2, heads2, static_cast<uint64_t>(d.total_pages)};
    const uint64_t strides[4] = {heads2 * 256, 128, 256, ps * heads2 * 256};
    const uint32_t box[5] = {64, static_cast<uint32_t>(ps), 2, 2, 1};
    int32_t rc = cake::encode_tensor_map(&plan->tmap_k, c0, 5, dims, strides, box, true);
    if (rc) return rc;
    plan->tmap_v = plan->tmap_k;
    return CAKE_OK;
  }
  const uint64_t hk = d.kv_heads;
  const uint64_t dims[5] = {64, ps, 2, hk, static_cast<uint64_t>(d.total_pages)};
  const uint64_t strides[4] = {hk * 256, 128, 256, ps * hk * 256};
  const uint32_t box[5] = {64, static_cast<uint32_t>(ps), 2, 1, 1};
  int32_t rc = cake::encode_tensor_map(&plan->tmap_k, c0, 5, dims, strides, box, true);
  if (rc) return rc;
  return cake::encode_tensor_map(&plan->tmap_v, c1, 5, dims, strides, box, true);
}
}  // namespace

extern "C" {

int32_t cake_rpa_create(const cake_rpa_desc* desc, cake_rpa** out) {
  if (!desc || !out) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_rpa_create: null argument");
  const cake_rpa_desc& d = *desc;
  if (d.num_seqs <= 0 || d.q_heads <= 0 || d.kv_heads <= 0 || d.total_pages <= 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: num_seqs, q_heads, kv_heads and total_pages must be positive");
  if (d.num_q_tokens != d.num_seqs)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa: only pure decode (one query token per sequence) is lowered; got %d tokens for %d sequences",
                d.num_q_tokens, d.num_seqs);
  if (d.q_heads % d.kv_heads != 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: q_heads %d must be a multiple of kv_heads %d", d.q_heads, d.kv_heads);
  if (d.q_heads / d.kv_heads > 16)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa: at most 16 query heads per KV head, got %d", d.q_heads / d.kv_heads);
  if (d.head_dim <= 0 || d.head_dim > 128 || d.head_dim % 8 != 0)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa: head_dim must be a multiple of 8 up to 128, got %d", d.head_dim);
  if (d.cache_layout == CAKE_RPA_CACHE_FUSED) {
    if (d.head_dim_padded != 128)
      return fail(CAKE_ERR_UNSUPPORTED, "rpa: fused cache rows must be padded to 128, got %d", d.head_dim_padded);
  } else if (d.cache_layout == CAKE_RPA_CACHE_SEPARATE) {
    if (d.head_dim != 128)
      return fail(CAKE_ERR_UNSUPPORTED, "rpa: separate K/V caches need head_dim 128, got %d", d.head_dim);
  } else {
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: unknown cache_layout %d", d.cache_layout);
  }
  int log2_ps = -1;
  for (int i = 0; i <= 5; ++i)
    if (d.page_size == (1 << i)) log2_ps = i;
  if (log2_ps < 0) return fail(CAKE_ERR_UNSUPPORTED, "rpa: page_size must be 1, 2, 4, 8, 16 or 32, got %d", d.page_size);
  if (d.table_layout != CAKE_RPA_TABLE_2D && d.table_layout != CAKE_RPA_TABLE_FLAT)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: unknown table_layout %d", d.table_layout);
  if (d.max_pages_per_seq <= 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: max_pages_per_seq (2-D row pitch, or flat table length) must be positive");
  if (d.total_pages >= INT32_MAX) return fail(CAKE_ERR_UNSUPPORTED, "rpa: total_pages must fit int32");
  if (d.bias_mode < 0 || d.bias_mode > 2) return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: bias_mode must be 0, 1 or 2");
  if (d.bias_mode != 0 && d.bias_extent <= 0) return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: bias_extent must be positive");
  if (d.bias_mode == 2 && d.rel_dim <= 0) return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: rel_dim must be positive");
  int chunk = d.kv_chunk_tokens == 0 ? 512 : d.kv_chunk_tokens;
  if (chunk < cake::kStageTokens || chunk % cake::kStageTokens != 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: kv_chunk_tokens must be a positive multiple of %d", cake::kStageTokens);

  cake_rpa* plan = new (std::nothrow) cake_rpa();
  if (!plan) return fail(CAKE_ERR_CUDA, "out of host memory");
  plan->d = d;
  plan->log2_ps = log2_ps;
  plan->chunk_tokens = chunk;
  int device = 0, major = 0;
  cudaError_t e = cudaGetDevice(&device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&plan->sm_count, cudaDevAttrMultiProcessorCount, device);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
  if (e != cudaSuccess) {
    delete plan;
    return fail(CAKE_ERR_CUDA, "no usable CUDA device: %s", cudaGetErrorString(e));
  }
  if (major != 10) {
    delete plan;
    return fail(CAKE_ERR_UNSUPPORTED, "libcake_b200 needs an sm_100 GPU, found compute capability %d.x", major);
  }
  // Upper bound on work items: every sequence can waste at most one partly filled chunk, and the
  // page table bounds the total number of tokens.
  const int64_t table_pages = d.table_layout == CAKE_RPA_TABLE_2D
                                  ? static_cast<int64_t>(d.num_seqs) * d.max_pages_per_seq
                                  : static_cast<int64_t>(d.max_pages_per_seq);
  const int64_t token_bound = table_pages * d.page_size;
  plan->max_items = (token_bound / chunk + d.num_seqs) * d.kv_heads;
  const int group = d.q_heads / d.kv_heads;
  rpa_layout_workspace(plan, group);
  int32_t rc = plan->status.ensure();
  if (rc) {
    delete plan;
    return rc;
  }
  *out = plan;
  return CAKE_OK;
}

int32_t cake_rpa_destroy(cake_rpa* plan) {
  if (!plan) return CAKE_OK;
  plan->status.release();
  delete plan;
  return CAKE_OK;
}

size_t cake_rpa_workspace_bytes(const cake_rpa* plan) { return plan ? plan->ws_bytes : 0; }

int32_t cake_rpa_launches_per_enqueue(const cake_rpa* plan) { return plan ? plan->launches : 0; }

int32_t cake_rpa_decode_enqueue(cake_rpa* plan, const void* q, const void* new_k, const void* new_v,
                                void* cache0, void* cache1, const int32_t* kv_lens,
                                const int32_t* page_table, const int32_t* cu_kv_lens,
                                const void* bias0, const void* bias1, void* out, void* workspace,
                                void* stream_v) {
  if (!plan || !q || !cache0 || !kv_lens || !page_table || !out || !workspace)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_rpa_decode_enqueue: null argument");
  const cake_rpa_desc& d = plan->d;
  if (d.cache_layout == CAKE_RPA_CACHE_SEPARATE && !cache1)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: separate cache layout needs a value cache");
  if (d.table_layout == CAKE_RPA_TABLE_FLAT && !cu_kv_lens)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: flat page table needs cu_kv_lens");
  if (d.update_cache && (!new_k || !new_v))
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: update_cache needs new_k and new_v");
  if (d.bias_mode == 1 && !bias0) return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: bias_mode 1 needs bias0");
  if (d.bias_mode == 2 && (!bias0 || !bias1)) return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: bias_mode 2 needs states and projection");
  if ((reinterpret_cast<uintptr_t>(cache0) | reinterpret_cast<uintptr_t>(cache1) |
       reinterpret_cast<uintptr_t>(workspace)) & 255)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: caches and workspace must be 256-byte aligned");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: q and out must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (cache0 != plan->last_c0 || cache1 != plan->last_c1) {
    int32_t rc = rpa_encode_maps(plan, cache0, cache1);
    if (rc) return rc;
    plan->last_c0 = cache0;
    plan->last_c1 = cache1;
  }
  cake::RpaParams p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.kv_lens = kv_lens;
  p.page_table = page_table;
  p.cu_kv_lens = cu_kv_lens;
  p.num_seqs = d.num_seqs;
  p.q_heads = d.q_heads;
  p.kv_heads = d.kv_heads;
  p.group = d.q_heads / d.kv_heads;
  p.head_dim = d.head_dim;
  p.page_size = d.page_size;
  p.log2_ps = plan->log2_ps;
  p.table_layout = d.table_layout;
  p.max_pages_per_seq = d.max_pages_per_seq;
  p.table_len = d.max_pages_per_seq;
  p.total_pages = static_cast<int32_t>(d.total_pages);
  p.fused = d.cache_layout == CAKE_RPA_CACHE_FUSED;
  p.chunk_tokens = plan->chunk_tokens;
  p.scale_log2 = d.sm_scale * 1.4426950408889634f;
  p.bias_mode = d.bias_mode;
  p.bias_extent = d.bias_extent;
  p.rel_dim = d.rel_dim;
  if (d.bias_mode == 1) p.bias = static_cast<const float*>(bias0);
  if (d.bias_mode == 2) {
    p.rel_states = static_cast<const __nv_bfloat16*>(bias0);
    p.rel_proj = static_cast<const __nv_bfloat16*>(bias1);
  }
  char* ws = static_cast<char*>(workspace);
  p.work_counter = reinterpret_cast<int32_t*>(ws);
  p.item_base = reinterpret_cast<int32_t*>(ws + plan->off_item_base);
  p.arrive = reinterpret_cast<int32_t*>(ws + plan->off_arrive);
  p.item_seq = reinterpret_cast<int32_t*>(ws + plan->off_item_seq);
  p.part_ml = reinterpret_cast<float*>(ws + plan->off_part_ml);
  p.part_o = reinterpret_cast<float*>(ws + plan->off_part_o);
  p.max_items = static_cast<int32_t>(plan->max_items > INT32_MAX ? INT32_MAX : plan->max_items);
  p.status = plan->status.dev;

  int launches = 0;
  cake::cake_rpa_plan_sm100<<<1, 256, 0, stream>>>(p);
  CAKE_CUDA_TRY(cudaGetLastError());
  ++launches;
  if (d.update_cache) {
    cake::cake_rpa_cache_update_sm100<<<d.num_seqs, 256, 0, stream>>>(
        p, static_cast<const __nv_bfloat16*>(new_k), static_cast<const __nv_bfloat16*>(new_v),
        static_cast<__nv_bfloat16*>(cache0), static_cast<__nv_bfloat16*>(cache1));
    CAKE_CUDA_TRY(cudaGetLastError());
    ++launches;
  }
  static bool configured = false;
  if (!configured) {
    CAKE_CUDA_TRY(cudaFuncSetAttribute(cake::cake_rpa_decode_sm100,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, cake::kRpaSmemBytes));
    configured = true;
  }
  cake::cake_rpa_decode_sm100<<<plan->sm_count, cake::kRpaThreads, cake::kRpaSmemBytes, stream>>>(
      plan->tmap_k, plan->tmap_v, p);
  CAKE_CUDA_TRY(cudaGetLastError());
  ++launches;
  plan->launches = launches;
  return CAKE_OK;
}

int32_t cake_rpa_status(cake_rpa* plan, void* stream_v, cake_status* out) {
  if (!plan || !out) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_rpa_status: null argument");
  int32_t rc = plan->status.read_and_clear(static_cast<cudaStream_t>(stream_v), out);
  if (rc) return rc;
  if (out->code == 1) return fail(CAKE_ERR_TIMEOUT, "rpa: bounded barrier wait ran out (block %d item %d stage %d)", out->detail0, out->detail1, out->detail2);
  if (out->code == 3) return fail(CAKE_ERR_DEVICE_CHECK, "rpa: page index out of range (sequence %d page slot %d value %d)", out->detail0, out->detail1, out->detail2);
  if (out->code == 4) return fail(CAKE_ERR_DEVICE_CHECK, "rpa: sequence metadata out of range (%d, %d, %d)", out->detail0, out->detail1, out->detail2);
  return CAKE_OK;
}

}  // extern "C"

// ====================================================================================== no-allocation variant
//
// cake_rpa_decode_static_scratch: the same decode, for hosts that are not allowed to allocate
// device memory -- a plugin running inside a serving engine that hands it fixed input / output
// buffers and owns the only allocator, or a loop whose memory pool is frozen after start-up, where
// a cudaMalloc would either be refused or would synchronise the whole device in the middle of
// serving. Such a host has nowhere to get the split-KV workspace from, so this variant keeps it in
// the array below, which is part of the library image: every GPU that loads the library holds
// CAKE_RPA_STATIC_SCRATCH_BYTES of it until the process exits.
//
// In host code the array's name is only a stand-in for the symbol, not a device address, so the
// address the kernels receive is looked up with cudaGetSymbolAddress, once per device, with that
// device current.

__device__ __align__(256) unsigned char g_cake_rpa_static_scratch[CAKE_RPA_STATIC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
void* g_static_scratch_address[kMaxDevices] = {};

// Derives the sizes cake_rpa_create would derive, into a caller-provided (stack) plan; validates
// the descriptor; touches no allocator.
int32_t rpa_prepare_without_allocation(const cake_rpa_desc& d, cake_rpa* plan) {
  if (d.num_seqs <= 0 || d.q_heads <= 0 || d.kv_heads <= 0 || d.total_pages <= 0 || d.total_pages >= INT32_MAX)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa (static scratch): num_seqs, q_heads, kv_heads, total_pages out of range");
  if (d.num_q_tokens != d.num_seqs)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa (static scratch): only pure decode is lowered");
  if (d.q_heads % d.kv_heads != 0 || d.q_heads / d.kv_heads > 16)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa (static scratch): q_heads must be 1..16 times kv_heads");
  if (d.head_dim <= 0 || d.head_dim > 128 || d.head_dim % 8 != 0)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa (static scratch): head_dim must be a multiple of 8 up to 128");
  if (d.cache_layout == CAKE_RPA_CACHE_FUSED ? d.head_dim_padded != 128
                                             : (d.cache_layout != CAKE_RPA_CACHE_SEPARATE || d.head_dim != 128))
    return fail(CAKE_ERR_UNSUPPORTED, "rpa (static scratch): cache rows must be 128 elements wide");
  int log2_ps = -1;
  for (int i = 0; i <= 5; ++i)
    if (d.page_size == (1 << i)) log2_ps = i;
  if (log2_ps < 0) return fail(CAKE_ERR_UNSUPPORTED, "rpa (static scratch): page_size must be a power of two up to 32");
  if ((d.table_layout != CAKE_RPA_TABLE_2D && d.table_layout != CAKE_RPA_TABLE_FLAT) || d.max_pages_per_seq <= 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa (static scratch): bad page-table layout or extent");
  if (d.bias_mode < 0 || d.bias_mode > 2 || (d.bias_mode != 0 && d.bias_extent <= 0) || (d.bias_mode == 2 && d.rel_dim <= 0))
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa (static scratch): bad bias description");
  const int chunk = d.kv_chunk_tokens == 0 ? 512 : d.kv_chunk_tokens;
  if (chunk < cake::kStageTokens || chunk % cake::kStageTokens != 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa (static scratch): kv_chunk_tokens must be a positive multiple of %d", cake::kStageTokens);
  plan->d = d;
  plan->log2_ps = log2_ps;
  plan->chunk_tokens = chunk;
  const int64_t table_pages = d.table_layout == CAKE_RPA_TABLE_2D
                                  ? static_cast<int64_t>(d.num_seqs) * d.max_pages_per_seq
                                  : static_cast<int64_t>(d.max_pages_per_seq);
  plan->max_items = (table_pages * d.page_size / chunk + d.num_seqs) * d.kv_heads;
  const int group = d.q_heads / d.kv_heads;
  rpa_layout_workspace(plan, group);
  return CAKE_OK;
}

}  // namespace

extern "C" int32_t cake_rpa_decode_static_scratch(const cake_rpa_desc* desc, const void* q,
                                                  const void* new_k, const void* new_v,
                                                  void* cache0, void* cache1, const int32_t* kv_lens,
                                                  const int32_t* page_table,
                                                  const int32_t* cu_kv_lens, const void* bias0,
                                                  const void* bias1, void* out,
                                                  int32_t* status_device, void* stream) {
  if (!desc) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_rpa_decode_static_scratch: null descriptor");
  cake_rpa plan;  // on the stack: no handle, nothing to destroy
  int32_t rc = rpa_prepare_without_allocation(*desc, &plan);
  if (rc) return rc;
  if (plan.ws_bytes > CAKE_RPA_STATIC_SCRATCH_BYTES)
    return fail(CAKE_ERR_UNSUPPORTED,
                "rpa (static scratch): this shape needs %zu bytes of split-KV scratch, the built-in array holds %u; "
                "use cake_rpa_decode_enqueue with a caller-provided workspace, or a larger kv_chunk_tokens",
                plan.ws_bytes, static_cast<unsigned>(CAKE_RPA_STATIC_SCRATCH_BYTES));
  int device = 0, major = 0;
  CAKE_CUDA_TRY(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) return fail(CAKE_ERR_UNSUPPORTED, "rpa (static scratch): device ordinal %d out of range", device);
  if (!g_static_scratch_address[device]) {
    // First call on this device: one-time set-up (do it before any stream capture begins).
    CAKE_CUDA_TRY(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
    if (major != 10) return fail(CAKE_ERR_UNSUPPORTED, "libcake_b200 needs an sm_100 GPU, found compute capability %d.x", major);
    void* address = nullptr;
    CAKE_CUDA_TRY(cudaGetSymbolAddress(&address, g_cake_rpa_static_scratch));
    if (!address) return fail(CAKE_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the static scratch");
    g_static_scratch_address[device] = address;
  }
  CAKE_CUDA_TRY(cudaDeviceGetAttribute(&plan.sm_count, cudaDevAttrMultiProcessorCount, device));
  plan.status.dev = status_device;  // caller-owned, may be null; never freed here
  rc = cake_rpa_decode_enqueue(&plan, q, new_k, new_v, cache0, cache1, kv_lens, page_table, cu_kv_lens,
                               bias0, bias1, out, g_static_scratch_address[device], stream);
  plan.status.dev = nullptr;
  return rc;
}
