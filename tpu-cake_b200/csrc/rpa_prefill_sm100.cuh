// Ragged paged attention for sequences with more than one query token (prefill and mixed batches),
// for sm_100a. Included by rpa_decode_sm100.cu (one translation unit: it shares RpaParams, the page
// lookup and the handle type with the decode path).
//
// What it replaces: the prefill / mixed branches of _owned_rpa_kernel_loop
// (src/tpu_cake/rpa_owned_kernel.py:85-960) selected by the `distribution` triple
// (src/tpu_cake/rpa_owned_kernel.py:58-67). The reference lowers only decode batches and has no
// oracle for longer query runs; semantics here are those of the wrapped kernel with causal=1: query
// token i of a sequence with q query tokens and kv_len cached tokens sits at position kv_len-q+i and
// sees positions 0..kv_len-q+i.
//
// Kernels
//   cake_rpa_ragged_update_sm100   writes the new K/V of EVERY query token at its position
//   cake_rpa_prefill_plan_sm100    cuts every sequence with index >= first_seq into 128-token query
//                                  tiles, later tiles (more visible KV) first
//   cake_rpa_prefill_sm100         persistent, one CTA per SM, warp-specialised:
//       warpgroup 0 / 1  softmax of query sub-tile 0 / 1 (one thread per query row; two query heads
//                        of one KV head share every KV tile)
//       warp 8           TMA producer: query tiles, then 64-token K/V stages gathered page by page.
//                        A stage is laid out [8-token group][K lo | K hi | V lo | V hi][8 rows][128 B]
//                        (lo / hi = the two 64-element halves of a 128-wide row): every 8-token group
//                        is one 4 KiB box of the fused cache, and the groups are a uniform 4 KiB apart,
//                        which is what the tcgen05 shared-memory descriptors need; no multicast
//       warp 9           tcgen05.mma issuer: S = Q K^T (128x64, K-major operands) and PV = P V
//                        (128x128, V consumed in place as an MN-major operand) into TMEM
//     S is read from TMEM with tcgen05.ld (a thread owns a row, so the row maximum and sum need no
//     shuffles), P goes back through shared memory in the 128-byte-swizzled K-major layout, and the
//     output accumulates in TMEM over all KV steps; it is read, rescaled and written back
//     (tcgen05.ld / tcgen05.st) only when a row maximum has moved by more than 2^8.
#pragma once

namespace cake {

constexpr int kPfThreads = 384;
constexpr int kPfTileQ = 128;
constexpr int kPfTileKv = 64;
constexpr int kPfStages = 3;
constexpr int kPfQBytes = kPfTileQ * 256;        // one sub-tile of queries: [2 halves][128 rows][128 B]
constexpr int kPfStageBytes = kPfTileKv * 512;   // [8 groups][K lo | K hi | V lo | V hi][8 rows][128 B]
constexpr int kPfGroupBytes = 4096;             // one 8-token group of a stage
constexpr int kPfPBytes = kPfTileQ * 128;        // P sub-tile: [128 rows][64 bf16]
constexpr int kPfSmemBytes = 2 * kPfQBytes + kPfStages * kPfStageBytes + 4 * kPfPBytes + 1024 + 1024;
constexpr uint32_t kPfTmemCols = 512;            // S0 @0, S1 @64, PV0 @128, PV1 @256
constexpr long long kPfBarrierBudget = 2000000000ll;
constexpr float kPfRescale = 8.f;                // log2 units the row maximum may lag before O is rescaled

struct PrefillParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int32_t* kv_lens;
  const int32_t* cu_q_lens;
  int32_t first_seq;       // sequences [first_seq, num_seqs) are handled here
  int32_t sub;             // query heads per work item: 2 when the GQA group is even, else 1
  int32_t heads_items;     // q_heads / sub
  int32_t* work_counter;
  int32_t* entry_count;    // number of (sequence, query tile) entries
  int4* entries;           // {sequence, first query row of the tile, q_len, kv_len}
  int32_t max_entries;
  int32_t num_q_tokens;
  RpaParams r;             // page table, layout, scale, status
};

#ifdef CAKE_PF_TIMING
// Development aid (off by default): cycles each role of every CTA spends blocked in its waits.
// Slots per CTA: 0 softmax wait S, 1 softmax wait PV, 2 softmax total, 3 softmax steps,
// 4 MMA wait K/V, 5 MMA wait S free, 6 MMA wait P, 7 MMA total, 8 producer wait slot, 9 producer total.
__device__ unsigned long long g_pf_timing[256 * 16];
#define PF_T0() const long long pf_t0_ = clock64()
#define PF_ADD(slot, cond) do { if (cond) g_pf_timing[blockIdx.x * 16 + (slot)] += clock64() - pf_t0_; } while (0)
#define PF_COUNT(slot, cond) do { if (cond) g_pf_timing[blockIdx.x * 16 + (slot)] += 1; } while (0)
#else
#define PF_T0() do {} while (0)
#define PF_ADD(slot, cond) do {} while (0)
#define PF_COUNT(slot, cond) do {} while (0)
#endif

__device__ __forceinline__ bool pf_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  while (true) {
    for (int i = 0; i < 32; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - start > kPfBarrierBudget) return false;
  }
}

// New K/V rows [num_q_tokens, kv_heads, head_dim] into the cache: token i of a sequence with q
// query tokens goes to position kv_len - q + i (for one query token: kv_len - 1, as
// src/tpu_cake/workloads/inkling_rpa.py:518-534). One CTA per query token.
__global__ void cake_rpa_ragged_update_sm100(PrefillParams pp, const __nv_bfloat16* new_k,
                                             const __nv_bfloat16* new_v, __nv_bfloat16* cache0,
                                             __nv_bfloat16* cache1) {
  const RpaParams& p = pp.r;
  const int t = blockIdx.x;
  int lo = 0, hi = p.num_seqs;  // largest s with cu_q[s] <= t
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (pp.cu_q_lens[mid] <= t) lo = mid; else hi = mid;
  }
  const int s = lo;
  const int q_len = pp.cu_q_lens[s + 1] - pp.cu_q_lens[s];
  const int i = t - pp.cu_q_lens[s];
  const int pos = p.kv_lens[s] - q_len + i;
  if (i >= q_len) return;  // tokens past the last sequence
  if (pos < 0) {
    if (threadIdx.x == 0) rpa_record(p.status, 4, s, p.kv_lens[s], q_len);
    return;
  }
  const int page = rpa_page_lookup(p, s, pos >> p.log2_ps);
  if (page < 0 || page >= p.total_pages) {
    if (threadIdx.x == 0) rpa_record(p.status, 3, s, pos >> p.log2_ps, page);
    return;
  }
  const int slot = pos & (p.page_size - 1);
  for (int e = threadIdx.x; e < p.kv_heads * 2 * 128; e += blockDim.x) {
    const int d = e & 127;
    const int kv = (e >> 7) & 1;
    const int h = e >> 8;
    const __nv_bfloat16* src = kv ? new_v : new_k;
    const __nv_bfloat16 val = d < p.head_dim ? src[(static_cast<size_t>(t) * p.kv_heads + h) * p.head_dim + d]
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

// Entry table of the prefill kernel. Tiles are emitted by distance from the end of their sequence
// (the last tile of every sequence first): later tiles see more KV, so the long items start first.
// Also checks that sequences before first_seq have exactly one query token each.
__global__ void __launch_bounds__(256) cake_rpa_prefill_plan_sm100(PrefillParams pp) {
  const RpaParams& p = pp.r;
  __shared__ int s_max_tiles;
  if (threadIdx.x == 0) {
    s_max_tiles = 0;
    *pp.work_counter = 0;
  }
  __syncthreads();
  int local_max = 0;
  for (int s = threadIdx.x; s < p.num_seqs; s += blockDim.x) {
    const int q_len = pp.cu_q_lens[s + 1] - pp.cu_q_lens[s];
    const int len = p.kv_lens[s];
    if (q_len < 0 || len < q_len || (s < pp.first_seq && q_len != 1) || pp.cu_q_lens[s + 1] > pp.num_q_tokens)
      rpa_record(p.status, 4, s, len, q_len);
    else if (s >= pp.first_seq)
      local_max = max(local_max, (q_len + kPfTileQ - 1) / kPfTileQ);
  }
  atomicMax(&s_max_tiles, local_max);
  __syncthreads();
  if (threadIdx.x != 0) return;
  int n = 0;
  for (int r = 0; r < s_max_tiles; ++r) {
    for (int s = pp.first_seq; s < p.num_seqs; ++s) {
      const int q_len = pp.cu_q_lens[s + 1] - pp.cu_q_lens[s];
      const int len = p.kv_lens[s];
      if (q_len <= 0 || len < q_len) continue;
      const int tiles = (q_len + kPfTileQ - 1) / kPfTileQ;
      if (tiles <= r) continue;
      if (n < pp.max_entries) pp.entries[n] = make_int4(s, (tiles - 1 - r) * kPfTileQ, q_len, len);
      ++n;
    }
  }
  if (n > pp.max_entries) {
    rpa_record(p.status, 4, n, pp.max_entries, 2);
    n = pp.max_entries;
  }
  *pp.entry_count = n;
}

__device__ __forceinline__ float pf_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 64-bit shared-memory descriptor from its two words.
__device__ __forceinline__ uint64_t pf_desc(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

__device__ __forceinline__ float pf_max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

__device__ __forceinline__ void pf_setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 208;" ::: "memory"); }
__device__ __forceinline__ void pf_setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 88;" ::: "memory"); }

__global__ void __launch_bounds__(kPfThreads, 1)
    cake_rpa_prefill_sm100(const __grid_constant__ CUtensorMap tmap_q,
                           const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const PrefillParams pp) {
  const RpaParams& p = pp.r;
  extern __shared__ uint8_t pf_smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pf_smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_smem = smem;                                     // [2 sub-tiles][2 halves][128][128 B]
  uint8_t* kv_smem = q_smem + 2 * kPfQBytes;                  // [stages][8 groups][4 atoms][8 rows][128 B]
  uint8_t* p_smem = kv_smem + kPfStages * kPfStageBytes;      // [2 sub-tiles][2 buffers][128][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + 4 * kPfPBytes);
  uint64_t* q_full = bars;              // [1]
  uint64_t* kv_full = bars + 1;         // [stages]
  uint64_t* kv_empty = kv_full + kPfStages;
  uint64_t* s_full = kv_empty + kPfStages;  // [2]
  uint64_t* p_full = s_full + 2;            // [2 sub-tiles][2 P buffers]
  uint64_t* pv_full = p_full + 4;           // [2 sub-tiles][2 P buffers]
  uint64_t* s_free = pv_full + 4;           // [2]
  uint64_t* drain_bar = s_free + 2;         // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  volatile int32_t* item_slot = reinterpret_cast<volatile int32_t*>(tmem_base_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < kPfStages; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(smem_u32(&s_full[g]), 1);
      mbar_init(smem_u32(&p_full[2 * g]), 128);
      mbar_init(smem_u32(&p_full[2 * g + 1]), 128);
      mbar_init(smem_u32(&pv_full[2 * g]), 1);
      mbar_init(smem_u32(&pv_full[2 * g + 1]), 1);
      mbar_init(smem_u32(&s_free[g]), 128);
    }
    mbar_init(smem_u32(drain_bar), 1);
    *abort_flag = 0;
    fence_mbar_init();
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(tmem_base_slot), kPfTmemCols);
    tmem_relinquish();
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;
  const int total_items = min(*pp.entry_count, pp.max_entries) * pp.heads_items;
  const int sub = pp.sub;

  // Running positions that persist across work items (every role that uses one advances it the
  // same way): K/V stages produced / consumed, KV steps processed (phase of s_full / p_full /
  // pv_full), query loads issued.
  uint32_t kv_pos = 0, step_total = 0, q_issued = 0;

  struct Item {
    int id, seq, q0, kv_len, head0, kvh, prior, rows, kv_needed, n_steps, q_tok0;
  };
  // Claims the next work item for the whole CTA. One thread decides (next item, or -1 after an
  // abort) so that every thread leaves its loop in the same iteration. The barrier also separates
  // items: when it opens, every role has finished the previous one, so the query and P buffers and
  // all TMEM columns are free.
  auto next_item = [&](uint32_t iter, Item& it) -> bool {
    if (threadIdx.x == 0) item_slot[iter & 1] = *abort_flag ? -1 : atomicAdd(pp.work_counter, 1);
    named_bar_sync(1, kPfThreads);
    const int id = item_slot[iter & 1];
    if (id < 0 || id >= total_items) return false;
    const int4 entry = __ldg(pp.entries + id / pp.heads_items);
    const int hi = id % pp.heads_items;
    it.id = id;
    it.seq = entry.x;
    it.q0 = entry.y;
    it.kv_len = entry.w;
    it.head0 = hi * sub;                        // first query head of the item
    it.kvh = it.head0 / p.group;                // its KV head
    it.prior = entry.w - entry.z;               // cached tokens before the first query token
    it.rows = min(kPfTileQ, entry.z - entry.y);
    it.kv_needed = it.prior + it.q0 + it.rows;  // positions any row of the tile can see
    it.n_steps = (it.kv_needed + kPfTileKv - 1) / kPfTileKv;
    it.q_tok0 = __ldg(pp.cu_q_lens + it.seq) + it.q0;
    return true;
  };
  Item it;

  if (warp < 8) {
    pf_setmaxnreg_inc();
    if (warp < 4 * sub) {
      // ---------------------------------------------------------------- softmax warpgroups
      const int g = warp >> 2;
      const int quarter = warp & 3;
      const int row = quarter * 32 + lane;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
      const uint32_t t_s = t_lane + g * 64;
      const uint32_t t_pv = t_lane + 128 + g * 128;
      uint8_t* p_rows = p_smem + g * 2 * kPfPBytes + row * 128;  // this thread's row in P buffer 0
      const float scale = p.scale_log2;  // positive: checked on the host
      for (uint32_t iter = 0; next_item(iter, it); ++iter) {
        PF_T0();
        const int limit = min(it.prior + it.q0 + row, it.kv_len - 1);  // last position this row sees
        // Running maximum (log2 domain, scaled) and sum of this thread's row. The output row itself
        // accumulates in TMEM across all KV steps; it is rescaled only when the maximum moves by more
        // than kPfRescale, so the exponentials below are bounded by 2^kPfRescale instead of 1.
        float m_run = kNegBig, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < it.n_steps; ++j) {
          {
            PF_T0();
            ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&s_full[g]), step_total & 1u, abort_flag));
            PF_ADD(0, threadIdx.x == 0);
            PF_COUNT(3, threadIdx.x == 0);
          }
          if (!ok) {
            if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 500 + g);
            *abort_flag = 1;
            break;
          }
          tcgen05_fence_after();
          uint32_t v[64];
          {
            uint32_t lo[32], hi[32];
            tmem_ld_32x32b_x32(t_s, lo);
            tmem_ld_32x32b_x32(t_s + 32, hi);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              v[c] = lo[c];
              v[32 + c] = hi[c];
            }
          }
          tcgen05_fence_before();
          mbar_arrive(smem_u32(&s_free[g]));  // S is in registers: the next S = Q K^T may overwrite it
          // P is double-buffered: this step writes buffer t & 1, which PV(t-2) read. Its barrier
          // completes every other step, so the wait below names exactly that completion.
          const uint32_t t = step_total;
          uint8_t* p_row = p_rows + (t & 1u) * kPfPBytes;
          if (j >= 2) {
            PF_T0();
            ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_full[2 * g + (t & 1u)]), ((t >> 1) & 1u) ^ 1u, abort_flag));
            PF_ADD(1, threadIdx.x == 0);
            if (!ok) {
              if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 700 + g);
              *abort_flag = 1;
              break;
            }
          }
          const int pos0 = j * kPfTileKv;
          // Only the steps that cross the row's causal limit (or the end of the sequence) mask.
          if (__any_sync(0xffffffffu, pos0 + kPfTileKv - 1 > limit)) {
#pragma unroll
            for (int c = 0; c < 64; ++c)
              if (pos0 + c > limit) v[c] = 0xff800000u;  // -inf
          }
          float mr = __uint_as_float(v[0]);
#pragma unroll
          for (int c = 1; c + 1 < 64; c += 2) mr = pf_max3(mr, __uint_as_float(v[c]), __uint_as_float(v[c + 1]));
          mr = fmaxf(mr, __uint_as_float(v[63]));
          const float mx = mr * scale;
          float alpha = 1.f;
          if (mx > m_run + kPfRescale) {
            alpha = pf_exp2(m_run - mx);
            m_run = mx;
          }
          // Rare: the accumulator is read and rewritten once PV(t-1) is complete; PV(t) is issued
          // only after p_full below.
          if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
            ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_full[2 * g + ((t - 1u) & 1u)]), ((t - 1u) >> 1) & 1u, abort_flag));
            if (!ok) {
              if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 800 + g);
              *abort_flag = 1;
              break;
            }
            tcgen05_fence_after();
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint32_t acc[32];
              tmem_ld_32x32b_x32(t_pv + c * 32, acc);
              tmem_ld_wait();
#pragma unroll
              for (int e = 0; e < 32; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
              tmem_st_32x32b_x32(t_pv + c * 32, acc);
            }
            tmem_st_wait();
          }
          // ---- P = exp2(S * scale - max) as bf16 into shared memory (K-major, 128-byte swizzle)
          const float neg_m = -m_run;
          float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
          for (int chunk = 0; chunk < 8; ++chunk) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int c = chunk * 8 + e * 2;
              const float a = pf_exp2(fmaf(__uint_as_float(v[c]), scale, neg_m));
              const float b = pf_exp2(fmaf(__uint_as_float(v[c + 1]), scale, neg_m));
              sum0 += a;
              sum1 += b;
              w[e] = pack_bf16(a, b);
            }
            *reinterpret_cast<uint4*>(p_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
          l_run = l_run * alpha + (sum0 + sum1);
          fence_proxy_async_smem();   // P written through the generic proxy, read by the tensor core
          tcgen05_fence_before();     // TMEM reads and writes above are ordered before the next MMAs
          // One barrier per P buffer: the softmax may run up to two steps ahead of the issuer, which a
          // single barrier's phase parity could not tell apart.
          mbar_arrive(smem_u32(&p_full[2 * g + (t & 1u)]));
          ++step_total;
        }
        if (ok) {
          // The last PV of the item.
          const uint32_t last = step_total - 1u;
          ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_full[2 * g + (last & 1u)]), (last >> 1) & 1u, abort_flag));
          if (!ok) {
            if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 600 + g);
            *abort_flag = 1;
          }
        }
        if (ok) {
          tcgen05_fence_after();
          const float inv = 1.f / l_run;
          __nv_bfloat16* dst = pp.out + (static_cast<size_t>(it.q_tok0 + row) * p.q_heads + it.head0 + g) * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t acc[32];
            tmem_ld_32x32b_x32(t_pv + c * 32, acc);
            tmem_ld_wait();
            if (row < it.rows) {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                uint4 piece;
                piece.x = pack_bf16(__uint_as_float(acc[e * 8 + 0]) * inv, __uint_as_float(acc[e * 8 + 1]) * inv);
                piece.y = pack_bf16(__uint_as_float(acc[e * 8 + 2]) * inv, __uint_as_float(acc[e * 8 + 3]) * inv);
                piece.z = pack_bf16(__uint_as_float(acc[e * 8 + 4]) * inv, __uint_as_float(acc[e * 8 + 5]) * inv);
                piece.w = pack_bf16(__uint_as_float(acc[e * 8 + 6]) * inv, __uint_as_float(acc[e * 8 + 7]) * inv);
                *reinterpret_cast<uint4*>(dst + c * 32 + e * 8) = piece;
              }
            }
          }
          tcgen05_fence_before();  // the accumulator reads are ordered before the next item's MMAs
        }
        PF_ADD(2, threadIdx.x == 0);
      }
    } else {
      // second warpgroup without a role (odd GQA group): only takes part in the item barrier
      for (uint32_t iter = 0; next_item(iter, it); ++iter) {
      }
    }
  } else {
    pf_setmaxnreg_dec();
    if (warp == 8) {
      // ---------------------------------------------------------------- TMA producer
      // Boxes: with pages of 8 tokens or more, one box is an 8-token group (K and V of the KV head,
      // both halves: 4 KiB of the fused cache, or 2 KiB from each of the separate caches); smaller
      // pages fill the four atoms of a group row by row, one box per page and atom.
      const int tb = min(p.page_size, 8);
      const int log2_tb = min(p.log2_ps, 3);
      const int boxes = kPfTileKv >> log2_tb;
      const bool wide = p.page_size >= 8;
      for (uint32_t iter = 0; next_item(iter, it); ++iter) {
        PF_T0();
        if (lane == 0) {
          mbar_arrive_expect_tx(smem_u32(q_full), static_cast<uint32_t>(sub * kPfQBytes));
          for (int g = 0; g < sub; ++g)
            for (int half = 0; half < 2; ++half)
              tma_load_2d(smem_u32(q_smem + g * kPfQBytes + half * (kPfQBytes / 2)), &tmap_q, smem_u32(q_full),
                          (it.head0 + g) * 128 + half * 64, it.q_tok0);
          ++q_issued;
        }
        __syncwarp();
        // Page ids are read 64 table slots at a time (two per lane) and the next 64 are requested
        // while the current ones are in use, so no stage waits for a table read of its own.
        const int pages_needed = (it.kv_needed + p.page_size - 1) >> p.log2_ps;
        const long long table_base = p.table_layout == CAKE_RPA_TABLE_2D
                                         ? static_cast<long long>(it.seq) * p.max_pages_per_seq
                                         : static_cast<long long>(p.cu_kv_lens[it.seq] >> p.log2_ps);
        const long long table_end = p.table_layout == CAKE_RPA_TABLE_2D ? table_base + p.max_pages_per_seq
                                                                        : static_cast<long long>(p.table_len);
        auto load_window = [&](int base_slot, int (&w)[2]) {
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int slot = base_slot + lane + 32 * r;
            int page = p.total_pages;  // out-of-range coordinate: the TMA unit fills the box with zeros
            if (slot < pages_needed) {
              const long long idx = table_base + slot;
              page = (idx >= 0 && idx < table_end) ? __ldg(p.page_table + idx) : -1;
              if (page < 0 || page >= p.total_pages) {
                rpa_record(p.status, 3, it.seq, slot, page);
                page = p.total_pages;
              }
            }
            w[r] = page;
          }
        };
        int win_base = 0;
        int win_cur[2], win_nxt[2];
        load_window(0, win_cur);
        load_window(64, win_nxt);
        for (int j = 0; j < it.n_steps; ++j) {
          const uint32_t stage = kv_pos % kPfStages;
          const uint32_t parity = (kv_pos / kPfStages) & 1u;
          const int first_slot = (j * kPfTileKv) >> p.log2_ps;
          if (first_slot >= win_base + 64) {  // a stage never straddles two windows
            win_base += 64;
            win_cur[0] = win_nxt[0];
            win_cur[1] = win_nxt[1];
            load_window(win_base + 64, win_nxt);
          }
          int my_page[2];
          int my_off[2];
#pragma unroll
          for (int rep = 0; rep < 2; ++rep) {
            const int b = lane + rep * 32;
            const int tok = j * kPfTileKv + b * tb;
            const int rel = (tok >> p.log2_ps) - win_base;  // 0..63 for the boxes of this stage
            const int from_lo = __shfl_sync(0xffffffffu, win_cur[0], rel & 31);
            const int from_hi = __shfl_sync(0xffffffffu, win_cur[1], rel & 31);
            const bool live = b < boxes && tok < it.kv_needed;
            my_page[rep] = live ? ((rel & 32) ? from_hi : from_lo) : p.total_pages;
            my_off[rep] = tok & (p.page_size - 1);
          }
          bool slot_free;
          {
            PF_T0();
            slot_free = __all_sync(0xffffffffu, pf_wait(smem_u32(&kv_empty[stage]), parity ^ 1u, abort_flag));
            PF_ADD(8, lane == 0);
          }
          if (!slot_free) {
            if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 100 + j);
            *abort_flag = 1;
            break;
          }
          const uint32_t bar = smem_u32(&kv_full[stage]);
          if (lane == 0) mbar_arrive_expect_tx(bar, kPfStageBytes);
          __syncwarp();
          const uint32_t sbase = smem_u32(kv_smem + stage * kPfStageBytes);
          const int hk = p.fused ? 2 * it.kvh : it.kvh;
          const int hv = p.fused ? 2 * it.kvh + 1 : it.kvh;
#pragma unroll
          for (int rep = 0; rep < 2; ++rep) {
            const int b = lane + rep * 32;
            if (b < boxes) {
              const int tok_in_stage = b * tb;
              const uint32_t gbase = sbase + static_cast<uint32_t>((tok_in_stage >> 3) * kPfGroupBytes);
              if (wide) {
                if (p.fused) {
                  tma_load_5d(gbase, &tmap_k, bar, 0, my_off[rep], 0, hk, my_page[rep]);
                } else {
                  tma_load_5d(gbase, &tmap_k, bar, 0, my_off[rep], 0, hk, my_page[rep]);
                  tma_load_5d(gbase + 2048, &tmap_v, bar, 0, my_off[rep], 0, hv, my_page[rep]);
                }
              } else {
                const uint32_t dst = gbase + static_cast<uint32_t>((tok_in_stage & 7) * 128);
                tma_load_5d(dst, &tmap_k, bar, 0, my_off[rep], 0, hk, my_page[rep]);
                tma_load_5d(dst + 1024, &tmap_k, bar, 0, my_off[rep], 1, hk, my_page[rep]);
                tma_load_5d(dst + 2048, &tmap_v, bar, 0, my_off[rep], 0, hv, my_page[rep]);
                tma_load_5d(dst + 3072, &tmap_v, bar, 0, my_off[rep], 1, hv, my_page[rep]);
              }
            }
          }
          __syncwarp();
          ++kv_pos;
        }
        PF_ADD(9, lane == 0);
      }
    } else if (warp == 9) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(kPfTileQ, kPfTileKv, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(kPfTileQ, 128, 0, 1);
      // Shared-memory descriptors, split into the low word (address field, which changes per MMA)
      // and the high word (stride field, version, swizzle mode: constant per operand kind).
      //   Q and P: K-major, 8-row groups 1 KiB apart.
      //   K tile:  K-major, 8-token groups 4 KiB apart; the second 64 elements of a row are the next atom.
      //   V tile:  [token][d] MN-major: the two 64-wide halves 1 KiB apart (leading offset), 8-token
      //            groups 4 KiB apart (stride offset); a K step of 16 tokens is two groups.
      const uint32_t desc_hi_1024 = static_cast<uint32_t>(umma_desc_sw128(0, 16, 1024) >> 32);
      const uint32_t desc_hi_k = static_cast<uint32_t>(umma_desc_sw128(0, 16, kPfGroupBytes) >> 32);
      const uint32_t desc_hi_v = static_cast<uint32_t>(umma_desc_sw128(0, 1024, kPfGroupBytes) >> 32);
      const uint32_t desc_q_lo = static_cast<uint32_t>(umma_desc_sw128(smem_u32(q_smem), 16, 1024));
      const uint32_t desc_p_lo = static_cast<uint32_t>(umma_desc_sw128(smem_u32(p_smem), 16, 1024));
      const uint32_t desc_k_lo = static_cast<uint32_t>(umma_desc_sw128(smem_u32(kv_smem), 16, kPfGroupBytes));
      const uint32_t desc_v_lo = static_cast<uint32_t>(umma_desc_sw128(smem_u32(kv_smem + 2048), 1024, kPfGroupBytes));
      for (uint32_t iter = 0; next_item(iter, it); ++iter) {
        PF_T0();
        int where = 200;
        // Waits for stage `pos`, then zeroes its V rows at or beyond kv_len (page tails may hold
        // anything; 0 * NaN would poison the product) before the tensor core reads them.
        auto stage_ready = [&](uint32_t pos, int j) -> bool {
          {
            PF_T0();
            const bool arrived = __all_sync(0xffffffffu, pf_wait(smem_u32(&kv_full[pos % kPfStages]), (pos / kPfStages) & 1u, abort_flag));
            PF_ADD(4, lane == 0);
            if (!arrived) return false;
          }
          const int first_bad = max(it.kv_len - j * kPfTileKv, 0);
          if (first_bad < kPfTileKv) {
            uint8_t* v_base = kv_smem + (pos % kPfStages) * kPfStageBytes + 2048;  // V lo of group 0
            for (int e = lane; e < (kPfTileKv - first_bad) * 16; e += 32) {
              const int row = first_bad + (e >> 4);
              const int piece = e & 15;
              *reinterpret_cast<uint4*>(v_base + (row >> 3) * kPfGroupBytes + (piece >> 3) * 1024 + (row & 7) * 128 +
                                        (piece & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async_smem();
          }
          __syncwarp();
          return true;
        };
        // Descriptors are built once (see above the item loop); per MMA only the 14-bit address
        // field moves, by an addition to the low word. The issuing thread shares its scheduler with
        // two softmax warps, so every instruction it does not execute is tensor time gained.
        auto issue_qk = [&](int g, uint32_t pos) {
          const uint32_t k_lo = desc_k_lo + (pos % kPfStages) * (kPfStageBytes >> 4);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t a_lo = desc_q_lo + g * (kPfQBytes >> 4) + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
            const uint32_t b_lo = k_lo + (((ks >> 2) * 1024 + (ks & 3) * 32) >> 4);
            tcgen05_mma_bf16(tmem_base + g * 64, pf_desc(a_lo, desc_hi_1024), pf_desc(b_lo, desc_hi_k), idesc_qk, ks != 0 ? 1u : 0u);
          }
          tcgen05_commit(smem_u32(&s_full[g]));
        };
        bool ok = __all_sync(0xffffffffu, pf_wait(smem_u32(q_full), iter & 1u, abort_flag));
        if (ok) ok = stage_ready(kv_pos, 0);
        if (ok) {
          tcgen05_fence_after();
          if (lane == 0)
            for (int g = 0; g < sub; ++g) issue_qk(g, kv_pos);
          __syncwarp();
          for (int j = 0; j < it.n_steps && ok; ++j) {
            if (j + 1 < it.n_steps) {
              where = 300;
              ok = stage_ready(kv_pos + 1, j + 1);
              if (!ok) break;
            }
            // Next S first: it only needs the softmax warps to have taken the current S into
            // registers, so Q K^T of step j+1 runs under the softmax of step j.
            if (j + 1 < it.n_steps) {
              for (int g = 0; g < sub; ++g) {
                where = 350 + g;
                PF_T0();
                ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&s_free[g]), step_total & 1u, abort_flag));
                PF_ADD(5, lane == 0);
                if (!ok) break;
                tcgen05_fence_after();
                if (lane == 0) issue_qk(g, kv_pos + 1);
                __syncwarp();
              }
              if (!ok) break;
            }
            for (int g = 0; g < sub; ++g) {
              where = 400 + g;
              PF_T0();
              ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&p_full[2 * g + (step_total & 1u)]), (step_total >> 1) & 1u, abort_flag));
              PF_ADD(6, lane == 0);
              if (!ok) break;
              tcgen05_fence_after();
              if (lane == 0) {
                const uint32_t buf = step_total & 1u;
                const uint32_t a_lo = desc_p_lo + (g * 2 + buf) * (kPfPBytes >> 4);
                const uint32_t b_lo = desc_v_lo + (kv_pos % kPfStages) * (kPfStageBytes >> 4);
                tcgen05_mma_bf16(tmem_base + 128 + g * 128, pf_desc(a_lo, desc_hi_1024), pf_desc(b_lo, desc_hi_v), idesc_pv, j != 0 ? 1u : 0u);
#pragma unroll
                for (int ks = 1; ks < 4; ++ks)
                  tcgen05_mma_bf16(tmem_base + 128 + g * 128, pf_desc(a_lo + ((ks * 32) >> 4), desc_hi_1024),
                                   pf_desc(b_lo + ((ks * 2 * kPfGroupBytes) >> 4), desc_hi_v), idesc_pv, 1u);
                tcgen05_commit(smem_u32(&pv_full[2 * g + buf]));
              }
              __syncwarp();
            }
            if (!ok) break;
            if (lane == 0) tcgen05_commit(smem_u32(&kv_empty[kv_pos % kPfStages]));
            __syncwarp();
            ++kv_pos;
            ++step_total;
          }
        }
        if (!ok) {
          if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, where);
          *abort_flag = 1;
        }
        __syncwarp();
        PF_ADD(7, lane == 0);
      }
    } else {
      // warps 10 and 11 have no role: they only take part in the item barrier
      for (uint32_t iter = 0; next_item(iter, it); ++iter) {
      }
    }
  }

  // ---- orderly exit
  __syncthreads();
  if (*abort_flag) {
    if (warp == 8 && lane == 0) {
      // loads already issued must land before shared memory is released
      if (q_issued) mbar_wait_bounded(smem_u32(q_full), (q_issued - 1) & 1u, 200000000ll);
      for (uint32_t back = 0; back < kPfStages && back < kv_pos; ++back) {
        const uint32_t pos = kv_pos - 1 - back;
        mbar_wait_bounded(smem_u32(&kv_full[pos % kPfStages]), (pos / kPfStages) & 1u, 200000000ll);
      }
    }
    if (warp == 9 && lane == 0) {
      tcgen05_commit(smem_u32(drain_bar));
      mbar_wait_bounded(smem_u32(drain_bar), 0, 200000000ll);
    }
    __syncthreads();
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kPfTmemCols);
  }
}

}  // namespace cake
