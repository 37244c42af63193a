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
//   cake_rpa_plan_sm100      one CTA: cuts every sequence into chunks and builds the work-item
//                            table (full chunks first, remainders last); resets the work counter
//   cake_rpa_cache_update_sm100  optional: writes each sequence's new K/V at position kv_len-1
//   cake_rpa_decode_sm100    persistent; every WARP (6 per CTA) is an independent worker with its
//                            own 2-stage shared-memory ring of 32-token stages. A work item is (sequence, KV head,
//                            chunk of the KV range). Pages are gathered through the page table
//                            with one TMA box per page (128-byte swizzle, never multicast); all
//                            query heads of the KV head share the page (GQA: each page is read
//                            once per KV head). The MMAs are issued with the KV side as the
//                            16-row operand and the query-head group (up to 8 heads) as the
//                            8-wide operand: S^T = K Q^T and O^T = V^T P^T on mma.sync m16n8k16,
//                            P^T obtained from the S^T accumulators with movmatrix; online softmax
//                            in f32 with warp shuffles.
//                            Loads run ahead into the next work item so the ring never drains.
//   cake_rpa_combine_sm100   one warp per (sequence, query head): merges the split-KV partials
//                            (m, l, o) in chunk order and writes bf16.
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
#ifndef CAKE_RPA_STAGE_TOKENS
#define CAKE_RPA_STAGE_TOKENS 32
#endif
constexpr int kStageTokens = CAKE_RPA_STAGE_TOKENS;  // 16 or 32
constexpr int kGroups16 = kStageTokens / 16;
static_assert(kStageTokens == 16 || kStageTokens == 32, "stage is one or two 16-token MMA groups");
constexpr int kRowBytes = 256;                                // one token of one head: 128 bf16
constexpr int kStageBytes = kStageTokens * 2 * kRowBytes;     // K and V: 16 KiB
constexpr int kQBufBytes = 8 * kRowBytes;                     // staged query rows of one work item
constexpr int kRpaSmemBytes = kRpaWarps * (kRpaStages * kStageBytes + kQBufBytes) + 1024 + 256;
constexpr long long kRpaBarrierBudget = 2000000000ll;
constexpr float kNegBig = -1.0e30f;

struct RpaParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  __nv_bfloat16* out_peers[CAKE_MAX_WORLD];  // every destination of an output row (own buffer first)
  int32_t out_count;
  const int32_t* kv_lens;
  const int32_t* page_table;
  const int32_t* cu_kv_lens;
  int32_t num_seqs, q_heads, kv_heads, group, head_dim;
  int32_t page_size, log2_ps;
  int32_t box_tokens, log2_box;  // tokens per TMA box: min(page_size, stage tokens)
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
  int32_t* tail_cs;    // [num_seqs] queue index of the sequence's remainder chunk, -1 if none
  int32_t* item_base;  // [num_seqs + 1] first full chunk of every sequence; [num_seqs] = total pairs
  int4* item_desc;     // [sum of chunk counts] {sequence, first token, kv_len, first pair of the sequence}
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

// kv_lens[s] if the page table can hold that many tokens, else 0: a length that is negative or
// larger than the table's room for the sequence (the 2-D table's row, or the rest of the flat index
// array) would walk into another sequence's pages, so every kernel treats such a sequence as empty
// and its output rows are left untouched. The planning kernels report it through the status word
// (code 4); the reference rejects the same inputs on the host
// (src/tpu_cake/rpa_lowering.py:94-104).
__device__ __forceinline__ int rpa_checked_len(const RpaParams& p, int s) {
  const int len = p.kv_lens[s];
  if (len <= 0) return 0;
  const long long pages = (static_cast<long long>(len) + p.page_size - 1) >> p.log2_ps;
  if (p.table_layout == CAKE_RPA_TABLE_2D) return pages <= p.max_pages_per_seq ? len : 0;
  const int start = p.cu_kv_lens[s];
  return (start >= 0 && (start >> p.log2_ps) + pages <= p.table_len) ? len : 0;
}

// Builds the work-item table. Every sequence is cut into chunks of chunk_tokens; the full chunks of
// all sequences come first in the queue and the shorter remainders last, so the kernel's tail is made
// of small items. item_base[s] = index of the sequence's first full chunk, tail_cs[s] = index of its
// remainder chunk (-1 if none), item_base[num_seqs] = total number of (sequence, chunk) pairs.
__global__ void __launch_bounds__(256) cake_rpa_plan_sm100(RpaParams p) {
  grid_dependency_trigger();  // the decode kernel may set itself up while this one runs
  __shared__ int s_full[256];
  __shared__ int s_tail[256];
  __shared__ int s_carry_full, s_carry_tail, s_total_full;
  const int tid = threadIdx.x;
  int local_full = 0;
  for (int s = tid; s < p.num_seqs; s += 256) {
    const int len = rpa_checked_len(p, s);
    if (len > 0) local_full += len / p.chunk_tokens;
    if (len != p.kv_lens[s]) rpa_record(p.status, 4, s, p.kv_lens[s], 0);
  }
  s_full[tid] = local_full;
  if (tid == 0) {
    s_carry_full = 0;
    s_carry_tail = 0;
    *p.work_counter = 0;
  }
  __syncthreads();
  for (int off = 128; off > 0; off >>= 1) {
    if (tid < off) s_full[tid] += s_full[tid + off];
    __syncthreads();
  }
  if (tid == 0) s_total_full = s_full[0];
  __syncthreads();
  const int total_full = s_total_full;
  for (int base = 0; base < p.num_seqs; base += 256) {
    const int s = base + tid;
    int nf = 0, ht = 0, len = 0;
    if (s < p.num_seqs) {
      len = rpa_checked_len(p, s);
      if (len > 0) {
        nf = len / p.chunk_tokens;
        ht = (len - nf * p.chunk_tokens) > 0 ? 1 : 0;
      }
    }
    __syncthreads();
    s_full[tid] = nf;
    s_tail[tid] = ht;
    __syncthreads();
    for (int off = 1; off < 256; off <<= 1) {
      int a = 0, b = 0;
      if (tid >= off) {
        a = s_full[tid - off];
        b = s_tail[tid - off];
      }
      __syncthreads();
      s_full[tid] += a;
      s_tail[tid] += b;
      __syncthreads();
    }
    if (s < p.num_seqs) {
      const int first_full = s_carry_full + s_full[tid] - nf;
      const int tail_pos = total_full + s_carry_tail + s_tail[tid] - ht;
      p.item_base[s] = first_full;
      p.tail_cs[s] = ht ? tail_pos : -1;
      if (static_cast<long long>(first_full + nf) * p.kv_heads <= p.max_items)
        for (int c = 0; c < nf; ++c) p.item_desc[first_full + c] = make_int4(s, c * p.chunk_tokens, len, first_full);
      if (ht && static_cast<long long>(tail_pos + 1) * p.kv_heads <= p.max_items)
        p.item_desc[tail_pos] = make_int4(s, nf * p.chunk_tokens, len, first_full);
    }
    __syncthreads();
    if (tid == 255) {
      s_carry_full += s_full[255];
      s_carry_tail += s_tail[255];
    }
    __syncthreads();
  }
  if (tid == 0) p.item_base[p.num_seqs] = total_full + s_carry_tail;
}

// Logical page slot -> physical page for token `tok` of sequence `s`.
__device__ __forceinline__ int rpa_page_lookup(const RpaParams& p, int s, int page_slot) {
  if (p.table_layout == CAKE_RPA_TABLE_2D) {
    if (page_slot < 0 || page_slot >= p.max_pages_per_seq) return -1;
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
  const int len = rpa_checked_len(p, s);
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
__device__ __forceinline__ uint32_t rpa_smem_off(int t, int c16, int kv, int box_tokens, int log2_box) {
  const int pg = t >> log2_box;
  const int tp = t & (box_tokens - 1);
  uint32_t off = static_cast<uint32_t>(pg * box_tokens * 512 + kv * box_tokens * 256 +
                                       (c16 >> 3) * box_tokens * 128 + tp * 128 + (c16 & 7) * 16);
  return off ^ (((off >> 7) & 7u) << 4);
}

// One unit of work of a warp: KV tokens [tok0, tok0 + ntok) of one (sequence, KV head).
struct RpaItem {
  int id, s, h, len, tok0, first_cs;  // first_cs: index of the sequence's first (sequence, chunk) pair
};

__device__ __forceinline__ int rpa_item_tokens(const RpaParams& p, const RpaItem& it) {
  return min(p.chunk_tokens, it.len - it.tok0);
}

__device__ __forceinline__ int rpa_item_chunks(const RpaParams& p, const RpaItem& it) {
  return (it.len + p.chunk_tokens - 1) / p.chunk_tokens;
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
  const int tb = p.box_tokens;                       // one box = tb tokens of one page
  const int boxes_per_stage = kStageTokens >> p.log2_box;
  const int ntok = rpa_item_tokens(p, it);
  const int rem = ntok - st * kStageTokens;
  const int nboxes = min(boxes_per_stage, (rem + tb - 1) >> p.log2_box);
  const int first = (st * kStageTokens) >> p.log2_ps;  // first page of the stage, relative to the item
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
  // Box `lane` of the stage: with pages no larger than a stage it is page first + lane; with larger
  // pages the stage is a single box somewhere inside page `first`.
  const int tok_in_item = st * kStageTokens + lane * tb;
  const int page = __shfl_sync(0xffffffffu, window_pages, (tok_in_item >> p.log2_ps) & 31);
  const int tok_off = tok_in_item & (ps - 1);
  if (lane == 0) mbar_arrive_expect_tx(bar, static_cast<uint32_t>(nboxes * tb * 512));
  __syncwarp();
  if (lane < nboxes) {
    const uint32_t dst = stage_smem + lane * tb * 512;
    if (p.fused) {
      tma_load_5d(dst, tmap_k, bar, 0, tok_off, 0, 2 * it.h, page);
    } else {
      tma_load_5d(dst, tmap_k, bar, 0, tok_off, 0, it.h, page);
      tma_load_5d(dst + tb * 256, tmap_v, bar, 0, tok_off, 0, it.h, page);
    }
  }
}

// Merges the split-KV partials of one (sequence, KV head) in chunk order and writes bf16 output.
// Lane c reads chunk c's (m, l).
__device__ __forceinline__ void rpa_merge(const RpaParams& p, int s, int h, int r, int n, int first_full, int tail, int lane) {
  const int n_full = n - (tail >= 0 ? 1 : 0);
  // Partial row of chunk c and query row r: chunk c is the c-th full chunk or the remainder.
  auto row_of = [&](int c, int r) {
    const size_t cs = c < n_full ? static_cast<size_t>(first_full + c) : static_cast<size_t>(tail);
    return (cs * p.kv_heads + h) * p.group + r;
  };
  {
    float m = kNegBig;
    for (int c0 = 0; c0 < n; c0 += 32) {
      const int c = c0 + lane;
      if (c < n) m = fmaxf(m, __ldcg(p.part_ml + row_of(c, r) * 2));
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float l = 0.f;
    float4 o = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = 0; c0 < n; c0 += 32) {
      const int c = c0 + lane;
      float w = 0.f;
      if (c < n) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(p.part_ml + row_of(c, r) * 2));
        w = exp2f(ml.x - m);
        l += ml.y * w;
      }
      const int cnt = min(32, n - c0);
      // Fixed chunk order; eight partial rows are requested together so their latencies overlap.
      for (int j0 = 0; j0 < cnt; j0 += 8) {
        float4 v[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int jj = min(j0 + u, cnt - 1);
          v[u] = __ldcg(reinterpret_cast<const float4*>(p.part_o + row_of(c0 + jj, r) * 128) + lane);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float wj = (j0 + u < cnt) ? __shfl_sync(0xffffffffu, w, (j0 + u) & 31) : 0.f;
          o.x += v[u].x * wj;
          o.y += v[u].y * wj;
          o.z += v[u].z * wj;
          o.w += v[u].w * wj;
        }
      }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
    const float inv = 1.f / l;
    if (lane * 4 < p.head_dim) {
      uint2 packed;
      packed.x = pack_bf16(o.x * inv, o.y * inv);
      packed.y = pack_bf16(o.z * inv, o.w * inv);
      const size_t at = (static_cast<size_t>(s) * p.q_heads + h * p.group + r) * p.head_dim + lane * 4;
      for (int o = 0; o < p.out_count; ++o) *reinterpret_cast<uint2*>(p.out_peers[o] + at) = packed;
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
  uint8_t* qbuf = smem + kRpaWarps * kRpaStages * kStageBytes + warp * kQBufBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kRpaWarps * (kRpaStages * kStageBytes + kQBufBytes)) +
                   warp * kRpaStages;
  if (lane == 0) {
    for (int s = 0; s < kRpaStages; ++s) mbar_init(smem_u32(&bars[s]), 1);
    fence_mbar_init();
    if (warp == 0) {
      prefetch_tensormap(&tmap_k);
      prefetch_tensormap(&tmap_v);
    }
  }
  // The query staging buffer holds 8 rows x 128 bf16; rows beyond the group and columns beyond
  // head_dim are never written again, so they stay zero.
  for (int i = lane; i < kQBufBytes / 16; i += 32)
    *reinterpret_cast<uint4*>(qbuf + i * 16) = make_uint4(0u, 0u, 0u, 0u);
  __syncwarp();

  // Everything above touched only this CTA's shared memory: it overlapped the kernels before this
  // one (launched with programmatic serialization). From here on their results are read.
  grid_dependency_wait();
  grid_dependency_trigger();
  const int total_items = p.item_base[p.num_seqs] * p.kv_heads;
  const int trow = lane >> 2;        // token (QK^T) or head-dim row (PV) this thread holds, +8 for c2/c3
  const int qrow = (lane & 3) * 2;   // query rows qrow, qrow + 1 of the accumulator fragments

  // Per-lane pieces of the ldmatrix addresses (stage-relative), fixed for the whole kernel. With
  // boxes of at least 8 tokens the 128-byte swizzle reduces to xor-ing the 16-byte chunk index
  // with (token & 7) == (lane & 7).
  const bool fast_addr = p.box_tokens >= 8;
  const int tb = p.box_tokens;
  const int tok_k = (lane & 7) + ((lane >> 3) & 1) * 8;  // K fragments: matrices (tok 0-7 | 8-15) x (chunk c | c+1)
  const int tok_v = (lane & 7) + (lane >> 4) * 8;        // V fragments: matrices (tok 0-7) x (c | c+1), (tok 8-15) x (c | c+1)
  uint32_t rowk[kGroups16], rowv[kGroups16];
#pragma unroll
  for (int g = 0; g < kGroups16; ++g) {
    const int tk = g * 16 + tok_k, tv = g * 16 + tok_v;
    rowk[g] = static_cast<uint32_t>((tk >> p.log2_box) * tb * 512 + (tk & (tb - 1)) * 128);
    rowv[g] = static_cast<uint32_t>((tv >> p.log2_box) * tb * 512 + tb * 256 + (tv & (tb - 1)) * 128);
  }
  const uint32_t dhi = static_cast<uint32_t>(tb * 128);      // second 64-element half of a row
  const uint32_t yk = static_cast<uint32_t>(((lane >> 4) ^ (lane & 7)) << 4);
  const uint32_t yv = static_cast<uint32_t>((((lane >> 3) & 1) ^ (lane & 7)) << 4);

  // The warp streams stages through its ring continuously: `consume_pos` counts stages computed,
  // `issue_pos` stages whose loads were issued; loads run ahead across the boundary into the next
  // work item so the ring never drains between items.
  //
  // Everything that costs a round trip to L2 is split into steps taken one per stage iteration, so
  // the round trip overlaps a stage of work instead of stalling the warp:
  //   next-item pipeline  ni_state 0 -> 1 queue atomic issued -> 2 descriptor load issued ->
  //                       3 item decoded, query rows being copied to smem  (4 = queue empty)
  RpaItem cur, nxt;
  int ni_state = 0, ni_raw = 0;
  int4 ni_desc = make_int4(0, 0, 0, 0);
  int cur_issued = 0, nxt_issued = 0;
  int cur_window = -1, nxt_window = -1, cur_pages = 0, nxt_pages = 0;
  uint32_t issue_pos = 0, consume_pos = 0;

  auto step_next_item = [&]() {
    if (ni_state == 0) {
      if (lane == 0) ni_raw = atomicAdd(p.work_counter, 1);
      ni_state = 1;
    } else if (ni_state == 1) {
      const int id = __shfl_sync(0xffffffffu, ni_raw, 0);
      if (id >= total_items) {
        ni_state = 4;
      } else if (id >= p.max_items) {
        if (lane == 0) rpa_record(p.status, 4, id, p.max_items, 1);
        ni_state = 4;
      } else {
        nxt.id = id;
        ni_desc = __ldg(p.item_desc + id / p.kv_heads);
        ni_state = 2;
      }
    } else if (ni_state == 2) {
      nxt.s = ni_desc.x;
      nxt.tok0 = ni_desc.y;
      nxt.len = ni_desc.z;
      nxt.first_cs = ni_desc.w;
      nxt.h = nxt.id % p.kv_heads;
      nxt_issued = 0;
      nxt_window = -1;
      // Copy the item's query rows into the staging buffer (16-byte pieces, XOR-swizzled by row).
      const int pieces = p.head_dim >> 3;
      const __nv_bfloat16* qsrc = p.q + (static_cast<size_t>(nxt.s) * p.q_heads + nxt.h * p.group) * p.head_dim;
      for (int i = lane; i < p.group * pieces; i += 32) {
        const int r = i / pieces, ck = i - r * pieces;
        const uint32_t dst = smem_u32(qbuf + r * 256 + ((ck ^ (r & 7)) << 4));
        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(qsrc + r * p.head_dim + ck * 8) : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      ni_state = 3;
    }
  };
  while (ni_state < 3) step_next_item();  // cold start: claim and decode the first item
  bool alive = true;

  while (ni_state == 3 && alive) {
    // ---- switch to the claimed item; its query rows are (or are about to be) in the staging buffer
    cur = nxt;
    cur_issued = nxt_issued;
    cur_window = nxt_window;
    cur_pages = nxt_pages;
    ni_state = 0;
    const int h = cur.h, s = cur.s, len = cur.len, tok0 = cur.tok0;
    const int ntok = rpa_item_tokens(p, cur);
    const int nstages = (ntok + kStageTokens - 1) / kStageTokens;
    const int n_chunks = rpa_item_chunks(p, cur);

    // ---- query fragments as the B operand: S^T[token, query row] = K[token, :] . Q[query row, :]
    uint32_t qb[8][2];
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncwarp();
    {
      const int r = lane & 7;
#pragma unroll
      for (int k2 = 0; k2 < 4; ++k2) {  // one x4 load covers two 16-wide k steps
        const int ck = k2 * 4 + (lane >> 3);
        ldmatrix_x4(smem_u32(qbuf + r * 256 + ((ck ^ r) << 4)), qb[2 * k2][0], qb[2 * k2][1], qb[2 * k2 + 1][0],
                    qb[2 * k2 + 1][1]);
      }
    }
    __syncwarp();

    float oacc[8][4];  // O^T: tile i holds head-dim rows i*16 + trow (+8) x query rows qrow, qrow+1
#pragma unroll
    for (int i = 0; i < 8; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
    float m_run[2] = {kNegBig, kNegBig};
    float l_run[2] = {0.f, 0.f};

    for (int st = 0; st < nstages; ++st) {
      // ---- top up the ring. A slot is refilled only after every lane finished reading it
      // (__syncwarp at the end of the previous stage) and a proxy fence orders those generic-proxy
      // reads before the async-proxy writes of the new TMA.
      fence_proxy_async_smem();
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
        if (ni_state != 3) break;
        const int nxt_stages = (rpa_item_tokens(p, nxt) + kStageTokens - 1) / kStageTokens;
        if (nxt_issued >= nxt_stages) break;
        rpa_issue_stage(p, &tmap_k, &tmap_v, nxt, nxt_issued, stage_smem, bar, lane, nxt_window, nxt_pages);
        ++nxt_issued;
        ++issue_pos;
      }
      // ---- one step of each bookkeeping pipeline; their memory traffic overlaps this stage
      step_next_item();
#ifdef CAKE_RPA_SYNC_FETCH
      while (ni_state < 3) step_next_item();
#endif

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
      const int n16 = (valid + 15) >> 4;  // 16-token groups to process

      // Zero V rows between the last valid token and the end of its 16-token group: their
      // contents are stale or uninitialised and 0 * NaN would poison the accumulator.
      if (valid < n16 * 16) {
        for (int t = valid; t < n16 * 16; ++t) {
          if (lane < 16) {
            const uint32_t off = rpa_smem_off(t, lane, 1, p.box_tokens, p.log2_box);
            asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(sbase + off), "r"(0u) : "memory");
          }
        }
        __syncwarp();
      }

      // ---- S^T = K Q^T: per 16-token group one accumulator tile [16 tokens x 8 query rows]
      float sacc[kGroups16][4];
#pragma unroll
      for (int g = 0; g < kGroups16; ++g) {
        sacc[g][0] = sacc[g][1] = sacc[g][2] = sacc[g][3] = 0.f;
        if (g < n16) {
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            uint32_t a[4];
            const uint32_t addr = fast_addr
                ? sbase + rowk[g] + (ks >> 2) * dhi + ((static_cast<uint32_t>((ks & 3) * 32)) ^ yk)
                : sbase + rpa_smem_off(g * 16 + tok_k, ks * 2 + (lane >> 4), 0, p.box_tokens, p.log2_box);
            ldmatrix_x4(addr, a[0], a[1], a[2], a[3]);
            mma_bf16_16816(sacc[g], a, qb[ks][0], qb[ks][1]);
          }
        }
      }

      // ---- scale, bias, mask (log2 domain); thread holds tokens trow, trow+8 of each group and
      //      query rows qrow (c0, c2) and qrow+1 (c1, c3)
      const int pos_base = tok0 + st * kStageTokens;
#pragma unroll
      for (int g = 0; g < kGroups16; ++g) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tk = g * 16 + trow + (e >> 1) * 8;
          float v = sacc[g][e] * p.scale_log2;
          if (p.bias_mode != 0) {
            const int row = qrow + (e & 1);
            const int pos = pos_base + tk;
            if (row < p.group && tk < valid) {
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
          }
          sacc[g][e] = (tk < valid) ? v : kNegBig;
        }
      }
      // ---- online softmax per query row: maxima over this thread's tokens, then over the 8 lanes
      //      that share the query-row pair (lane bits 2..4)
      float mx0 = kNegBig, mx1 = kNegBig;
#pragma unroll
      for (int g = 0; g < kGroups16; ++g) {
        mx0 = fmaxf(mx0, fmaxf(sacc[g][0], sacc[g][2]));
        mx1 = fmaxf(mx1, fmaxf(sacc[g][1], sacc[g][3]));
      }
#pragma unroll
      for (int off = 4; off < 32; off <<= 1) {
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, off));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, off));
      }
      const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
      const bool rescale = (mn0 != m_run[0]) || (mn1 != m_run[1]);
      const float al0 = exp2f(m_run[0] - mn0), al1 = exp2f(m_run[1] - mn1);
      m_run[0] = mn0;
      m_run[1] = mn1;
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int g = 0; g < kGroups16; ++g) {
        sacc[g][0] = exp2f(sacc[g][0] - mn0);
        sacc[g][1] = exp2f(sacc[g][1] - mn1);
        sacc[g][2] = exp2f(sacc[g][2] - mn0);
        sacc[g][3] = exp2f(sacc[g][3] - mn1);
        sum0 += sacc[g][0] + sacc[g][2];
        sum1 += sacc[g][1] + sacc[g][3];
      }
      l_run[0] = l_run[0] * al0 + sum0;
      l_run[1] = l_run[1] * al1 + sum1;
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          oacc[i][0] *= al0;
          oacc[i][1] *= al1;
          oacc[i][2] *= al0;
          oacc[i][3] *= al1;
        }
      }

      // ---- O^T += V^T P^T: P^T fragments come from the S^T accumulators through a warp-level
      //      8x8 transpose (movmatrix)
#pragma unroll
      for (int g = 0; g < kGroups16; ++g) {
        if (g < n16) {
          uint32_t pb0, pb1;
          const uint32_t lo = pack_bf16(sacc[g][0], sacc[g][1]);
          const uint32_t hi = pack_bf16(sacc[g][2], sacc[g][3]);
          asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb0) : "r"(lo));
          asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(pb1) : "r"(hi));
#pragma unroll
          for (int dt = 0; dt < 8; ++dt) {
            uint32_t a[4];
            const uint32_t addr = fast_addr
                ? sbase + rowv[g] + (dt >> 2) * dhi + ((static_cast<uint32_t>((dt & 3) * 32)) ^ yv)
                : sbase + rpa_smem_off(g * 16 + tok_v, dt * 2 + ((lane >> 3) & 1), 1, p.box_tokens, p.log2_box);
            ldmatrix_x4_trans(addr, a[0], a[1], a[2], a[3]);
            mma_bf16_16816(oacc[dt], a, pb0, pb1);
          }
        }
      }
      __syncwarp();
      ++consume_pos;
    }
    if (!alive) break;

    // ---- finish the item: row sums over the 8 lanes of each query-row pair, then output or partial
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], off);
      l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], off);
    }
    if (n_chunks == 1) {
      const float inv0 = 1.f / l_run[0], inv1 = 1.f / l_run[1];
      const size_t at0 = (static_cast<size_t>(s) * p.q_heads + h * p.group + qrow) * p.head_dim;
      for (int o = 0; o < p.out_count; ++o) {
        __nv_bfloat16* o0 = p.out_peers[o] + at0;
        __nv_bfloat16* o1 = o0 + p.head_dim;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int d = i * 16 + trow;
          if (qrow < p.group) {
            if (d < p.head_dim) o0[d] = __float2bfloat16_rn(oacc[i][0] * inv0);
            if (d + 8 < p.head_dim) o0[d + 8] = __float2bfloat16_rn(oacc[i][2] * inv0);
          }
          if (qrow + 1 < p.group) {
            if (d < p.head_dim) o1[d] = __float2bfloat16_rn(oacc[i][1] * inv1);
            if (d + 8 < p.head_dim) o1[d + 8] = __float2bfloat16_rn(oacc[i][3] * inv1);
          }
        }
      }
    } else {
      float* po = p.part_o + (static_cast<size_t>(cur.id) * p.group + qrow) * 128;
      float* pml = p.part_ml + (static_cast<size_t>(cur.id) * p.group + qrow) * 2;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int d = i * 16 + trow;
        if (qrow < p.group) {
          po[d] = oacc[i][0];
          po[d + 8] = oacc[i][2];
        }
        if (qrow + 1 < p.group) {
          po[128 + d] = oacc[i][1];
          po[128 + d + 8] = oacc[i][3];
        }
      }
      if (trow == 0) {
        if (qrow < p.group) *reinterpret_cast<float2*>(pml) = make_float2(m_run[0], l_run[0]);
        if (qrow + 1 < p.group) *reinterpret_cast<float2*>(pml + 2) = make_float2(m_run[1], l_run[1]);
      }
      // cake_rpa_combine_sm100 merges the partials of each (sequence, KV head) after this kernel.
    }

    while (ni_state < 3) step_next_item();  // short items may not have finished claiming the next one
  }

  if (!alive) {
    // A wait ran out: let loads already issued land before shared memory is released.
    asm volatile("cp.async.wait_all;" ::: "memory");
    for (uint32_t pos = consume_pos; pos < issue_pos; ++pos)
      mbar_wait_bounded(smem_u32(&bars[pos % kRpaStages]), (pos / kRpaStages) & 1u, 100000000ll);
  }
}

// One warp per (sequence, KV head, query row): merges its split-KV partials in chunk order.
__global__ void __launch_bounds__(128) cake_rpa_combine_sm100(const RpaParams p) {
  grid_dependency_wait();  // launched early; the partials are complete only when the decode kernel is
  const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= p.num_seqs * p.kv_heads * p.group) return;
  const int pair = unit / p.group;
  const int r = unit - pair * p.group;
  const int s = pair / p.kv_heads;
  const int h = pair - s * p.kv_heads;
  const int len = rpa_checked_len(p, s);
  const int n = len > 0 ? (len + p.chunk_tokens - 1) / p.chunk_tokens : 0;
  if (n > 1) rpa_merge(p, s, h, r, n, p.item_base[s], p.tail_cs[s], threadIdx.x & 31);
}

// After the decode and combine kernels have written this rank's output slice into every rank's
// gathered buffer: tell every rank (release at system scope, after the wait on the kernels before
// ordered the slice's stores before this kernel) and wait, bounded, until every rank has told us.
// Launched with programmatic stream serialization, so its launch latency hides behind the combine
// kernel; the wait below is where it meets it.
__global__ void cake_rpa_gather_sync_sm100(unsigned long long* const* flags_of, int world, int rank,
                                           unsigned long long epoch, int wait,
                                           unsigned long long budget_ns, int32_t* status) {
  grid_dependency_wait();
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(flags_of[r] + rank), "l"(epoch) : "memory");
  if (!wait) return;
  const unsigned long long start = global_timer_ns();
  while (ld_acquire_sys_u64(flags_of[rank] + r) < epoch) {
    if (global_timer_ns() - start > budget_ns) {
      rpa_record(status, 2, rank, r, 0);
      return;
    }
    __nanosleep(100);
  }
}

}  // namespace cake

#include "rpa_prefill_sm100.cuh"

// ====================================================================================== host

struct cake_rpa {
  cake_rpa_desc d;
  int sm_count = 0;
  int log2_ps = 0;
  int chunk_tokens = 0;
  int64_t max_items = 0;
  size_t off_item_base = 0, off_item_desc = 0, off_tail = 0, off_part_o = 0, off_part_ml = 0, ws_bytes = 0;
  cake::StatusWord status;
  const void* last_c0 = nullptr;
  const void* last_c1 = nullptr;
  CUtensorMap tmap_k, tmap_v;
  int launches = 0;
  // all-gather of outputs over peer memory (set for the duration of one gather enqueue)
  int gather_world = 0;
  void* gather_out[CAKE_MAX_WORLD] = {};
  unsigned long long gather_epoch = 0;
  unsigned long long** gather_flag_table = nullptr;  // device copy of the W flag-array pointers
  void* gather_flags_seen[CAKE_MAX_WORLD] = {};
  // mixed batches: the decode kernels run on the first `active_seqs` sequences (0 = all) and leave
  // the cache update to the ragged update kernel
  int active_seqs = 0;
  bool skip_update = false;
  size_t off_pf_entries = 0;
  int64_t max_pf_entries = 0;
  const void* last_q = nullptr;
  const void* last_pf_c0 = nullptr;
  const void* last_pf_c1 = nullptr;
  CUtensorMap tmap_q, tmap_pf_k, tmap_pf_v;
};

namespace {
using cake::fail;

// The opt-in to more than 48 KB of dynamic shared memory is an attribute of the (function, device)
// pair: remember per device ordinal whether it has been set.
template <typename Kernel>
int32_t opt_in_shared_memory(Kernel kernel, int bytes, bool (&configured)[64]) {
  int device = 0;
  CAKE_CUDA_TRY(cudaGetDevice(&device));
  const bool tracked = device >= 0 && device < 64;
  if (tracked && configured[device]) return CAKE_OK;
  CAKE_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
  if (tracked) configured[device] = true;
  return CAKE_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Workspace: [work counter | item_base | item_desc | tail_cs | partial (m,l) | partial o].
void rpa_layout_workspace(cake_rpa* plan, int group) {
  const cake_rpa_desc& d = plan->d;
  plan->off_item_base = 256;
  plan->off_item_desc = align_up(plan->off_item_base + sizeof(int32_t) * (d.num_seqs + 1), 256);
  plan->off_tail = align_up(plan->off_item_desc + 16 * (plan->max_items / d.kv_heads + 1), 256);
  plan->off_part_ml = align_up(plan->off_tail + sizeof(int32_t) * d.num_seqs, 256);
  plan->off_part_o = align_up(plan->off_part_ml + sizeof(float) * 2 * group * plan->max_items, 256);
  plan->off_pf_entries = align_up(plan->off_part_o + sizeof(float) * 128 * group * plan->max_items, 256);
  plan->max_pf_entries = (d.num_q_tokens + 127) / 128 + d.num_seqs;
  plan->ws_bytes = plan->off_pf_entries + 32 * static_cast<size_t>(plan->max_pf_entries);
}

int32_t rpa_encode_maps(cake_rpa* plan, const void* c0, const void* c1) {
  const cake_rpa_desc& d = plan->d;
  const uint64_t ps = d.page_size;
  const uint32_t tb = static_cast<uint32_t>(d.page_size < cake::kStageTokens ? d.page_size : cake::kStageTokens);
  if (d.cache_layout == CAKE_RPA_CACHE_FUSED) {
    const uint64_t heads2 = 2ull * d.kv_heads;
    const uint64_t dims[5] = {64, ps, 2, heads2, static_cast<uint64_t>(d.total_pages)};
    const uint64_t strides[4] = {heads2 * 256, 128, 256, ps * heads2 * 256};
    const uint32_t box[5] = {64, tb, 2, 2, 1};
    int32_t rc = cake::encode_tensor_map(&plan->tmap_k, c0, 5, dims, strides, box, true);
    if (rc) return rc;
    plan->tmap_v = plan->tmap_k;
    return CAKE_OK;
  }
  const uint64_t hk = d.kv_heads;
  const uint64_t dims[5] = {64, ps, 2, hk, static_cast<uint64_t>(d.total_pages)};
  const uint64_t strides[4] = {hk * 256, 128, 256, ps * hk * 256};
  const uint32_t box[5] = {64, tb, 2, 1, 1};
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
  if (d.num_q_tokens < d.num_seqs)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: %d query tokens for %d sequences", d.num_q_tokens, d.num_seqs);
  if (d.q_heads % d.kv_heads != 0)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: q_heads %d must be a multiple of kv_heads %d", d.q_heads, d.kv_heads);
  if (d.q_heads / d.kv_heads > 8)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa: at most 8 query heads per KV head, got %d", d.q_heads / d.kv_heads);
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
  // Library default of the split-KV chunk: 512 tokens (the chunk search on the 64-sequence decode:
  // 212 / 226 / 232 us for 512 / 256 / 1024). With one or two KV heads on this GPU -- a decode sharded
  // by KV head over many GPUs -- a work item carries so few bytes that the per-item costs show, and
  // 1024 measured 2-3 % faster than 512 (256 sequences of 1 Ki - 32 Ki tokens: 0.245 against 0.250 ms
  // with one head, 0.447 against 0.463 ms with two; 2048 and more lose to the tail of the queue).
  int chunk = d.kv_chunk_tokens == 0 ? (d.kv_heads <= 2 ? 1024 : 512) : d.kv_chunk_tokens;
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
  if (plan->gather_flag_table) cudaFree(plan->gather_flag_table);
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
  if (d.num_q_tokens != d.num_seqs && plan->active_seqs == 0)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa: the decode call takes one query token per sequence (got %d tokens for %d sequences); "
                "use cake_rpa_mixed_enqueue", d.num_q_tokens, d.num_seqs);
  const int num_seqs = plan->active_seqs ? plan->active_seqs : d.num_seqs;
  const bool update = d.update_cache && !plan->skip_update;
  if (d.cache_layout == CAKE_RPA_CACHE_SEPARATE && !cache1)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: separate cache layout needs a value cache");
  if (d.table_layout == CAKE_RPA_TABLE_FLAT && !cu_kv_lens)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: flat page table needs cu_kv_lens");
  if (update && (!new_k || !new_v))
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
  p.out_peers[0] = p.out;
  p.out_count = 1;
  if (plan->gather_world > 1) {
    p.out_count = plan->gather_world;
    for (int o = 0; o < plan->gather_world; ++o) p.out_peers[o] = static_cast<__nv_bfloat16*>(plan->gather_out[o]);
    p.out = p.out_peers[0];
  }
  p.kv_lens = kv_lens;
  p.page_table = page_table;
  p.cu_kv_lens = cu_kv_lens;
  p.num_seqs = num_seqs;
  p.q_heads = d.q_heads;
  p.kv_heads = d.kv_heads;
  p.group = d.q_heads / d.kv_heads;
  p.head_dim = d.head_dim;
  p.page_size = d.page_size;
  p.log2_ps = plan->log2_ps;
  p.box_tokens = d.page_size < cake::kStageTokens ? d.page_size : cake::kStageTokens;
  p.log2_box = plan->log2_ps < (cake::kStageTokens == 16 ? 4 : 5) ? plan->log2_ps : (cake::kStageTokens == 16 ? 4 : 5);
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
  p.tail_cs = reinterpret_cast<int32_t*>(ws + plan->off_tail);
  p.item_desc = reinterpret_cast<int4*>(ws + plan->off_item_desc);
  p.part_ml = reinterpret_cast<float*>(ws + plan->off_part_ml);
  p.part_o = reinterpret_cast<float*>(ws + plan->off_part_o);
  p.max_items = static_cast<int32_t>(plan->max_items > INT32_MAX ? INT32_MAX : plan->max_items);
  p.status = plan->status.dev;

  int launches = 0;
  cake::cake_rpa_plan_sm100<<<1, 256, 0, stream>>>(p);
  CAKE_CUDA_TRY(cudaGetLastError());
  ++launches;
  if (update) {
    cake::cake_rpa_cache_update_sm100<<<num_seqs, 256, 0, stream>>>(
        p, static_cast<const __nv_bfloat16*>(new_k), static_cast<const __nv_bfloat16*>(new_v),
        static_cast<__nv_bfloat16*>(cache0), static_cast<__nv_bfloat16*>(cache1));
    CAKE_CUDA_TRY(cudaGetLastError());
    ++launches;
  }
  {
    static bool configured[64] = {};
    int32_t arc = opt_in_shared_memory(cake::cake_rpa_decode_sm100, cake::kRpaSmemBytes, configured);
    if (arc) return arc;
  }
  // Decode and combine are launched with programmatic stream serialization: each may be scheduled
  // while its predecessor still runs and waits on the device (griddepcontrol.wait) before reading
  // what the predecessor wrote, so launch latency and set-up overlap the predecessor's tail.
  cudaLaunchAttribute overlap_attr;
  overlap_attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  overlap_attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config;
  memset(&config, 0, sizeof(config));
  config.stream = stream;
  config.attrs = &overlap_attr;
  config.numAttrs = 1;
  config.gridDim = dim3(plan->sm_count);
  config.blockDim = dim3(cake::kRpaThreads);
  config.dynamicSmemBytes = cake::kRpaSmemBytes;
  CAKE_CUDA_TRY(cudaLaunchKernelEx(&config, cake::cake_rpa_decode_sm100, plan->tmap_k, plan->tmap_v, p));
  ++launches;
  config.gridDim = dim3((num_seqs * d.q_heads + 3) / 4);
  config.blockDim = dim3(128);
  config.dynamicSmemBytes = 0;
  CAKE_CUDA_TRY(cudaLaunchKernelEx(&config, cake::cake_rpa_combine_sm100, p));
  ++launches;
  plan->launches = launches;
  return CAKE_OK;
}

int32_t cake_rpa_decode_allgather_enqueue(cake_rpa* plan, const void* q, const void* new_k,
                                          const void* new_v, void* cache0, void* cache1,
                                          const int32_t* kv_lens, const int32_t* page_table,
                                          const int32_t* cu_kv_lens, const void* bias0,
                                          const void* bias1, void* const* gathered,
                                          void* const* flags, int32_t world, int32_t rank,
                                          int32_t wait, void* workspace, void* stream_v) {
  if (!plan || !gathered || !flags) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_rpa_decode_allgather_enqueue: null argument");
  if (world < 1 || world > CAKE_MAX_WORLD || rank < 0 || rank >= world)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa all-gather: bad mesh world=%d rank=%d", world, rank);
  const cake_rpa_desc& d = plan->d;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const size_t slice_bytes = static_cast<size_t>(d.num_seqs) * d.q_heads * d.head_dim * 2;
  // Call n writes half n & 1 of every rank's buffer: a rank that is one call ahead of a peer
  // cannot overwrite what the peer's consumer of the previous call is still reading.
  const size_t half_offset = ((plan->gather_epoch + 1) & 1ull) * world * slice_bytes;
  // Own buffer first, so the local copy does not wait behind link traffic.
  for (int i = 0; i < world; ++i) {
    const int r = (rank + i) % world;
    if (!gathered[r] || !flags[r]) return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa all-gather: missing buffer of rank %d", r);
    plan->gather_out[i] = static_cast<char*>(gathered[r]) + half_offset + rank * slice_bytes;
  }
  if (!plan->gather_flag_table) {
    CAKE_CUDA_TRY(cudaMalloc(&plan->gather_flag_table, sizeof(void*) * CAKE_MAX_WORLD));
  }
  bool flags_changed = false;
  for (int r = 0; r < world; ++r) flags_changed |= plan->gather_flags_seen[r] != flags[r];
  if (flags_changed) {
    CAKE_CUDA_TRY(cudaMemcpyAsync(plan->gather_flag_table, flags, sizeof(void*) * world, cudaMemcpyHostToDevice, stream));
    for (int r = 0; r < world; ++r) plan->gather_flags_seen[r] = flags[r];
  }
  plan->gather_world = world;
  int32_t rc = cake_rpa_decode_enqueue(plan, q, new_k, new_v, cache0, cache1, kv_lens, page_table, cu_kv_lens, bias0, bias1,
                                       plan->gather_out[0], workspace, stream_v);
  plan->gather_world = 0;
  if (rc) return rc;
  plan->gather_epoch += 1;
  const unsigned long long budget_ns =
      (d.wait_budget_ms > 0 ? static_cast<unsigned long long>(d.wait_budget_ms) : 20000ull) * 1000000ull;
  cudaLaunchAttribute overlap_attr;
  overlap_attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  overlap_attr.val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t config;
  memset(&config, 0, sizeof(config));
  config.stream = stream;
  config.attrs = &overlap_attr;
  config.numAttrs = 1;
  config.gridDim = dim3(1);
  config.blockDim = dim3(32);
  CAKE_CUDA_TRY(cudaLaunchKernelEx(&config, cake::cake_rpa_gather_sync_sm100,
                                   static_cast<unsigned long long* const*>(plan->gather_flag_table), world, rank,
                                   plan->gather_epoch, wait, budget_ns, plan->status.dev));
  plan->launches += 1;
  return CAKE_OK;
}

int32_t cake_rpa_mixed_enqueue(cake_rpa* plan, const void* q, const void* new_k, const void* new_v,
                               void* cache0, void* cache1, const int32_t* kv_lens,
                               const int32_t* page_table, const int32_t* cu_kv_lens,
                               const int32_t* cu_q_lens, int32_t num_decode_seqs, void* out,
                               void* workspace, void* stream_v) {
  if (!plan || !q || !cache0 || !kv_lens || !page_table || !cu_q_lens || !out || !workspace)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_rpa_mixed_enqueue: null argument");
  const cake_rpa_desc& d = plan->d;
  if (num_decode_seqs < 0 || num_decode_seqs > d.num_seqs)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa mixed: num_decode_seqs %d outside [0, %d]", num_decode_seqs, d.num_seqs);
  if (d.head_dim != 128) return fail(CAKE_ERR_UNSUPPORTED, "rpa mixed: head_dim must be 128, got %d", d.head_dim);
  if (d.bias_mode != 0) return fail(CAKE_ERR_UNSUPPORTED, "rpa mixed: attention bias is lowered for decode batches only");
  if (!(d.sm_scale > 0.f)) return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa mixed: sm_scale must be positive");
  if (d.cache_layout != CAKE_RPA_CACHE_FUSED)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa mixed: ragged batches are lowered for the fused cache layout");
  if (d.cache_layout == CAKE_RPA_CACHE_SEPARATE && !cache1)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: separate cache layout needs a value cache");
  if (d.table_layout == CAKE_RPA_TABLE_FLAT && !cu_kv_lens)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: flat page table needs cu_kv_lens");
  if (d.update_cache && (!new_k || !new_v))
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: update_cache needs new_k and new_v");
  if ((reinterpret_cast<uintptr_t>(cache0) | reinterpret_cast<uintptr_t>(cache1) | reinterpret_cast<uintptr_t>(workspace)) & 255)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: caches and workspace must be 256-byte aligned");
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out)) & 15)
    return fail(CAKE_ERR_INVALID_ARGUMENT, "rpa: q and out must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const int group = d.q_heads / d.kv_heads;

  // Tensor maps: queries [tokens][q_heads*128] in boxes of 64 columns x 128 rows; caches below.
  if (q != plan->last_q) {
    const uint64_t dims[2] = {static_cast<uint64_t>(d.q_heads) * 128, static_cast<uint64_t>(d.num_q_tokens)};
    const uint64_t strides[1] = {static_cast<uint64_t>(d.q_heads) * 256};
    const uint32_t box[2] = {64, 128};
    int32_t rc = cake::encode_tensor_map(&plan->tmap_q, q, 2, dims, strides, box, true);
    if (rc) return rc;
    plan->last_q = q;
  }
  if (cache0 != plan->last_pf_c0 || cache1 != plan->last_pf_c1) {
    const uint64_t ps = d.page_size;
    const bool fused = d.cache_layout == CAKE_RPA_CACHE_FUSED;
    const uint64_t heads = fused ? 2ull * d.kv_heads : static_cast<uint64_t>(d.kv_heads);
    const uint64_t dims[5] = {64, ps, 2, heads, static_cast<uint64_t>(d.total_pages)};
    const uint64_t strides[4] = {heads * 256, 128, 256, ps * heads * 256};
    // Pages of 8 tokens or more: one box = an 8-token group of one head's K (or V) with both halves
    // of the row. Smaller pages: one box = one page of one half row.
    const bool wide = d.page_size >= 8;
    const uint32_t box[5] = {64, static_cast<uint32_t>(wide ? 8 : d.page_size), wide ? 2u : 1u, 1, 1};
    int32_t rc = cake::encode_tensor_map(&plan->tmap_pf_k, cache0, 5, dims, strides, box, true);
    if (rc) return rc;
    // V tiles are consumed 16 tokens per MMA: with pages of 16 tokens or more a V box is 16 tokens.
    const uint32_t box_v[5] = {64, static_cast<uint32_t>(d.page_size >= 16 ? 16 : box[1]), box[2], 1, 1};
    rc = cake::encode_tensor_map(&plan->tmap_pf_v, fused ? cache0 : cache1, 5, dims, strides, box_v, true);
    if (rc) return rc;
    plan->last_pf_c0 = cache0;
    plan->last_pf_c1 = cache1;
  }

  char* ws = static_cast<char*>(workspace);
  cake::PrefillParams pp;
  memset(&pp, 0, sizeof(pp));
  pp.q = static_cast<const __nv_bfloat16*>(q);
  pp.out = static_cast<__nv_bfloat16*>(out);
  pp.kv_lens = kv_lens;
  pp.cu_q_lens = cu_q_lens;
  pp.first_seq = num_decode_seqs;
  pp.paired = (d.q_heads / d.kv_heads) % 2 == 0 ? 1 : 0;
  pp.heads_items = pp.paired ? d.q_heads / 2 : d.q_heads;
  pp.work_counter = reinterpret_cast<int32_t*>(ws + 64);
  pp.entry_count = reinterpret_cast<int32_t*>(ws + 128);
  pp.entries = reinterpret_cast<int4*>(ws + plan->off_pf_entries);
  pp.max_entries = static_cast<int32_t>(plan->max_pf_entries);
  pp.num_q_tokens = d.num_q_tokens;
  cake::RpaParams& p = pp.r;
  p.kv_lens = kv_lens;
  p.page_table = page_table;
  p.cu_kv_lens = cu_kv_lens;
  p.num_seqs = d.num_seqs;
  p.q_heads = d.q_heads;
  p.kv_heads = d.kv_heads;
  p.group = group;
  p.head_dim = d.head_dim;
  p.page_size = d.page_size;
  p.log2_ps = plan->log2_ps;
  p.box_tokens = d.page_size;   // page_size <= 32 < one 64-token stage: one box per page and half row
  p.log2_box = plan->log2_ps;
  p.table_layout = d.table_layout;
  p.max_pages_per_seq = d.max_pages_per_seq;
  p.table_len = d.max_pages_per_seq;
  p.total_pages = static_cast<int32_t>(d.total_pages);
  p.fused = d.cache_layout == CAKE_RPA_CACHE_FUSED;
  p.scale_log2 = d.sm_scale * 1.4426950408889634f;
  p.status = plan->status.dev;

  int launches = 0;
  if (d.update_cache) {
    cake::cake_rpa_ragged_update_sm100<<<d.num_q_tokens, 256, 0, stream>>>(
        pp, static_cast<const __nv_bfloat16*>(new_k), static_cast<const __nv_bfloat16*>(new_v),
        static_cast<__nv_bfloat16*>(cache0), static_cast<__nv_bfloat16*>(cache1));
    CAKE_CUDA_TRY(cudaGetLastError());
    ++launches;
  }
  cake::cake_rpa_prefill_plan_sm100<<<1, 256, 0, stream>>>(pp);
  CAKE_CUDA_TRY(cudaGetLastError());
  ++launches;
  if (num_decode_seqs > 0) {
    // Decode sequences come first and own query tokens 0..num_decode_seqs-1 (checked by the plan
    // kernel above), so the decode kernels index q and out by sequence as in a pure decode batch.
    plan->active_seqs = num_decode_seqs;
    plan->skip_update = true;
    const int32_t rc = cake_rpa_decode_enqueue(plan, q, new_k, new_v, cache0, cache1, kv_lens, page_table, cu_kv_lens,
                                               nullptr, nullptr, out, workspace, stream_v);
    plan->active_seqs = 0;
    plan->skip_update = false;
    if (rc) return rc;
    launches += plan->launches;
  }
  if (num_decode_seqs < d.num_seqs) {
    static bool configured[64] = {};
    int32_t arc = opt_in_shared_memory(cake::cake_rpa_prefill_sm100, cake::kPfSmemBytes, configured);
    if (arc) return arc;
    cake::cake_rpa_prefill_sm100<<<plan->sm_count, cake::kPfThreads, cake::kPfSmemBytes, stream>>>(
        plan->tmap_q, plan->tmap_pf_k, plan->tmap_pf_v, pp);
    CAKE_CUDA_TRY(cudaGetLastError());
    ++launches;
  }
  plan->launches = launches;
  return CAKE_OK;
}

int32_t cake_rpa_status(cake_rpa* plan, void* stream_v, cake_status* out) {
  if (!plan || !out) return fail(CAKE_ERR_INVALID_ARGUMENT, "cake_rpa_status: null argument");
  int32_t rc = plan->status.read_and_clear(static_cast<cudaStream_t>(stream_v), out);
  if (rc) return rc;
  if (out->code == 2) return fail(CAKE_ERR_TIMEOUT, "rpa all-gather: rank %d never heard from rank %d", out->detail0, out->detail1);
  if (out->code == 1) return fail(CAKE_ERR_TIMEOUT, "rpa: bounded barrier wait ran out (block %d item %d stage %d)", out->detail0, out->detail1, out->detail2);
  if (out->code == 3) return fail(CAKE_ERR_DEVICE_CHECK, "rpa: page index out of range (sequence %d page slot %d value %d)", out->detail0, out->detail1, out->detail2);
  if (out->code == 4) return fail(CAKE_ERR_DEVICE_CHECK, "rpa: sequence metadata out of range (%d, %d, %d)", out->detail0, out->detail1, out->detail2);
  if (out->code == 5) return fail(CAKE_ERR_DEVICE_CHECK, "rpa: dynamic shared memory of block %d is not 1 KiB aligned (offset %d)", out->detail0, out->detail1);
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
  if (d.q_heads % d.kv_heads != 0 || d.q_heads / d.kv_heads > 8)
    return fail(CAKE_ERR_UNSUPPORTED, "rpa (static scratch): q_heads must be 1..8 times kv_heads");
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
