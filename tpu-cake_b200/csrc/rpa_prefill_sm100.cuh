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
//   cake_rpa_prefill_sm100         persistent, one CTA per SM; a work item is 128 query tokens of one
//                                  query head, walked over the KV range in steps of 128 tokens.
//       warps 0-7   softmax: two threads per query row (TMEM lane), one per 64-column half of a step,
//                   so the row maximum needs one exchange through shared memory and no shuffles.
//                   S comes out of TMEM with tcgen05.ld, P = exp2(S - max) goes back into TMEM
//                   (tcgen05.st, bf16 pairs, double-buffered) where the tensor core reads it as the
//                   A operand, so P never touches shared memory; the output row accumulates in TMEM
//                   over all steps and is read, rescaled and written back only when its maximum has
//                   moved by more than 2^8.
//       warps 8, 11 TMA producers of the query tile and of the K ring (3 slots), half a tile each
//       warp 10     TMA producer of the V ring (3 slots). K tiles are gathered page by page in boxes of
//                   one 8-token group (both 64-element halves of the row: 2 KiB), laid out
//                   [group][lo | hi][8 rows][128 B]: groups a uniform 2 KiB apart, which is what the
//                   tcgen05 shared-memory descriptor of a 128-token operand needs. V tiles are read
//                   16 tokens per MMA, so their boxes are 16 tokens (4 KiB) when pages allow: half
//                   as many copy instructions (each costs its issuing warp about 70 cycles).
//                   Never multicast.
//       warp 9      tcgen05.mma issuer: S = Q K^T (128x128x128, both operands K-major in shared
//                   memory) two steps ahead of the softmax, as soon as the softmax warps have taken
//                   the previous S into registers, and O += P V (128x128x128, P from TMEM, V consumed
//                   in place from shared memory as an MN-major operand) when P is written.
//     A 128-wide MMA keeps the tensor pipe busy for about 64 cycles, which is also what the issuing
//     thread needs per instruction; 64-wide steps were issue-bound.
#pragma once

namespace cake {

constexpr int kPfThreads = 384;
constexpr int kPfTileQ = 128;                    // query rows per work item (one query head)
constexpr int kPfTileKv = 128;                   // KV tokens per step
constexpr int kPfRing = 3;                       // slots of the K ring and of the V ring
constexpr int kPfQBytes = kPfTileQ * 256;        // queries: [2 halves][128 rows][128 B]
constexpr int kPfTileBytes = kPfTileKv * 256;    // a K or V tile: [16 groups][lo | hi][8 rows][128 B]
constexpr int kPfGroupBytes = 2048;              // one 8-token group of a K or V tile
constexpr int kPfTailBytes = 3072;               // barriers, TMEM slot, item slots, 2 KiB row-maximum exchange
constexpr int kPfSmemBytes = kPfQBytes + 2 * kPfRing * kPfTileBytes + kPfTailBytes;  // all a CTA may own
constexpr uint32_t kPfTmemCols = 512;            // S @0 (128 columns), O @128 (128), P buffers @256 and @320 (64 each)
constexpr uint32_t kPfTmemP = 256;
constexpr long long kPfBarrierBudget = 2000000000ll;
constexpr float kPfRescale = 8.f;                // log2 units the row maximum may lag before O is rescaled

struct PrefillParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int32_t* kv_lens;
  const int32_t* cu_q_lens;
  int32_t first_seq;       // sequences [first_seq, num_seqs) are handled here
  int32_t heads_items;     // work items per (sequence, query tile): one per query head
  int32_t* work_counter;
  int32_t* entry_count;    // number of (sequence, query tile) entries
  int4* entries;           // two per tile: {sequence, first query row, q_len, kv_len}, {first query token, first page-table slot, 0, 0}
  int32_t max_entries;
  int32_t num_q_tokens;
  RpaParams r;             // page table, layout, scale, status
};

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
  const int pos = rpa_checked_len(p, s) - q_len + i;
  if (i >= q_len) return;  // tokens past the last sequence
  if (pos < 0) {  // also: a length the page table cannot hold (checked length 0)
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
    const int len = rpa_checked_len(p, s);
    if (len != p.kv_lens[s] || q_len < 0 || len < q_len || (s < pp.first_seq && q_len != 1) || pp.cu_q_lens[s + 1] > pp.num_q_tokens)
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
      const int len = rpa_checked_len(p, s);
      if (q_len <= 0 || len < q_len) continue;
      const int tiles = (q_len + kPfTileQ - 1) / kPfTileQ;
      if (tiles <= r) continue;
      if (n < pp.max_entries) {
        const int q0 = (tiles - 1 - r) * kPfTileQ;
        const int table_base = p.table_layout == CAKE_RPA_TABLE_2D ? s * p.max_pages_per_seq : (p.cu_kv_lens[s] >> p.log2_ps);
        pp.entries[2 * n] = make_int4(s, q0, q_len, len);
        pp.entries[2 * n + 1] = make_int4(pp.cu_q_lens[s] + q0, table_base, 0, 0);  // saves two dependent loads per item
      }
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

__global__ void __launch_bounds__(kPfThreads, 1)
    cake_rpa_prefill_sm100(const __grid_constant__ CUtensorMap tmap_q,
                           const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const PrefillParams pp) {
  const RpaParams& p = pp.r;
  // The tiles need 1 KiB alignment (128-byte swizzle atoms) and the CTA uses every byte it may own,
  // so there is no slack to round the base up: the alignment is requested and checked.
  extern __shared__ __align__(1024) uint8_t pf_smem_raw[];
  uint8_t* smem = pf_smem_raw;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) rpa_record(p.status, 5, blockIdx.x, static_cast<int>(smem_u32(smem) & 1023u), 0);
    return;
  }
  uint8_t* q_smem = smem;                                  // [2 halves][128 rows][128 B]
  uint8_t* k_smem = q_smem + kPfQBytes;                    // [ring][16 groups][lo | hi][8 rows][128 B]
  uint8_t* v_smem = k_smem + kPfRing * kPfTileBytes;       // same
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + kPfRing * kPfTileBytes);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* k_full = bars + 1;             // [ring]
  uint64_t* k_empty = k_full + kPfRing;    // [ring]
  uint64_t* v_full = k_empty + kPfRing;    // [ring]
  uint64_t* v_empty = v_full + kPfRing;    // [ring]
  uint64_t* s_full = v_empty + kPfRing;    // [1]
  uint64_t* s_free = s_full + 1;           // [1]
  uint64_t* p_full = s_free + 1;           // [2 P buffers]
  uint64_t* pv_full = p_full + 2;          // [2 P buffers]
  uint64_t* drain_bar = pv_full + 2;       // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  volatile int32_t* item_slot = reinterpret_cast<volatile int32_t*>(tmem_base_slot + 2);  // [2]
  float* xchg = reinterpret_cast<float*>(tmem_base_slot + 4);  // [2 parities][2 column halves][128 rows]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < kPfRing; ++s) {
      mbar_init(smem_u32(&k_full[s]), 2);  // two producer warps, half a tile each
      mbar_init(smem_u32(&k_empty[s]), 1);
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
    }
    mbar_init(smem_u32(s_full), 1);
    mbar_init(smem_u32(s_free), 256);
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&p_full[b]), 256);
      mbar_init(smem_u32(&pv_full[b]), 1);
    }
    mbar_init(smem_u32(drain_bar), 1);
    *abort_flag = 0;
    item_slot[0] = atomicAdd(pp.work_counter, 1);
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

  // Running step count that persists across work items: every role advances it the same way. It
  // gives the ring slot (t % ring), the P buffer (t & 1) and every barrier phase.
  uint32_t step_total = 0;
  uint32_t loads_issued = 0;  // producers: tiles issued, for the orderly exit

  struct Item {
    int id, seq, q0, kv_len, head, kvh, prior, rows, kv_needed, n_steps, q_tok0, table_base;
  };
  // Hands the next work item to the whole CTA. One thread claims (an item, or -1 after an abort),
  // one item ahead, so that every thread leaves its loop in the same iteration. The barrier also
  // separates items: when it opens, every role has finished the previous one, so the query buffer
  // and all TMEM columns are free.
  auto next_item = [&](uint32_t iter, Item& it) -> bool {
    named_bar_sync(1, kPfThreads);
    const int id = item_slot[iter & 1];
    // The claim for the item after this one is issued now, so its latency hides under this item.
    if (threadIdx.x == 0) item_slot[(iter + 1) & 1] = *abort_flag ? -1 : atomicAdd(pp.work_counter, 1);
    if (id < 0 || id >= total_items) return false;
    const int4* entry_pair = pp.entries + 2 * (id / pp.heads_items);
    const int4 entry = __ldg(entry_pair);
    const int4 where = __ldg(entry_pair + 1);
    it.id = id;
    it.seq = entry.x;
    it.q0 = entry.y;
    it.kv_len = entry.w;
    it.head = id % pp.heads_items;
    it.kvh = it.head / p.group;
    it.prior = entry.w - entry.z;               // cached tokens before the first query token
    it.rows = min(kPfTileQ, entry.z - entry.y);
    it.kv_needed = it.prior + it.q0 + it.rows;  // positions any row of the tile can see
    it.n_steps = (it.kv_needed + kPfTileKv - 1) / kPfTileKv;
    it.q_tok0 = where.x;
    it.table_base = where.y;
    return true;
  };
  Item it;

  if (warp < 8) {
    // ---------------------------------------------------------------- softmax warps
    // Two threads per query row: warp w and warp w + 4 read the same TMEM lanes (32 (w & 3) ...) and
    // take the lower and upper 64 columns of S, P and O. The row maximum is combined through shared
    // memory once per step (a 64-thread named barrier per warp pair), so both threads derive the
    // same running maximum and the same rescale decisions; the row sums are combined at the end.
    const int quarter = warp & 3;
    const int half = warp >> 2;
    const int row = quarter * 32 + lane;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t t_s = t_lane + half * 64;
    const uint32_t t_o = t_lane + 128 + half * 64;
    const uint32_t t_p = t_lane + kPfTmemP + half * 32;  // this thread's 32 packed columns of P buffer 0
    const uint32_t pair_barrier = 2 + quarter;
    const float scale = p.scale_log2;  // positive: checked on the host
    for (uint32_t iter = 0; next_item(iter, it); ++iter) {
      const int limit = min(it.prior + it.q0 + row, it.kv_len - 1);  // last position this row sees
      // Running maximum (log2 domain, scaled) of the row and sum of this thread's columns. The
      // maximum is allowed to lag by kPfRescale, so the exponentials are bounded by 2^kPfRescale.
      float m_run = kNegBig, l_run = 0.f;
      bool ok = true;
      for (int j = 0; j < it.n_steps; ++j) {
        const uint32_t t = step_total;
        {
          ok = __all_sync(0xffffffffu, pf_wait(smem_u32(s_full), t & 1u, abort_flag));
        }
        if (!ok) {
          if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 500);
          *abort_flag = 1;
          break;
        }
        tcgen05_fence_after();
        uint32_t v[64];
        {
          uint32_t c0[32], c1[32];
          tmem_ld_32x32b_x32(t_s, c0);
          tmem_ld_32x32b_x32(t_s + 32, c1);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            v[c] = c0[c];
            v[32 + c] = c1[c];
          }
        }
        tcgen05_fence_before();
        mbar_arrive(smem_u32(s_free));  // S is in registers: the next S = Q K^T may overwrite it
        const int pos0 = j * kPfTileKv + half * 64;
        // Only the steps that cross the row's causal limit (or the end of the sequence) mask.
        if (__any_sync(0xffffffffu, pos0 + 63 > limit)) {
#pragma unroll
          for (int c = 0; c < 64; ++c)
            if (pos0 + c > limit) v[c] = 0xff800000u;  // -inf
        }
        float mr0 = __uint_as_float(v[0]), mr1 = __uint_as_float(v[1]);
#pragma unroll
        for (int c = 2; c + 3 < 64; c += 4) {
          mr0 = pf_max3(mr0, __uint_as_float(v[c]), __uint_as_float(v[c + 1]));
          mr1 = pf_max3(mr1, __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
        }
        const float mine = pf_max3(mr0, mr1, fmaxf(__uint_as_float(v[62]), __uint_as_float(v[63])));
        // Combine with the thread that holds the other 64 columns of this row.
        float* slot = xchg + (t & 1u) * 256;
        slot[half * 128 + row] = mine;
        named_bar_sync(pair_barrier, 64);
        const float mx = fmaxf(mine, slot[(half ^ 1) * 128 + row]) * scale;
        // P is double-buffered: this step writes buffer t & 1, which PV(t-2) read. Each buffer has
        // its own barriers, completing every other step, so a wait names exactly one completion
        // even though this role may run up to two steps ahead of the issuer.
        if (j >= 2) {
          ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_full[t & 1u]), ((t >> 1) & 1u) ^ 1u, abort_flag));
          if (!ok) {
            if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 700);
            *abort_flag = 1;
            break;
          }
        }
        float alpha = 1.f;
        if (mx > m_run + kPfRescale) {
          alpha = pf_exp2(m_run - mx);
          m_run = mx;
        }
        // Rare: the accumulator is read and rewritten once PV(t-1) is complete; PV(t) is issued
        // only after p_full below. Both threads of a row take the same decision.
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_full[(t - 1u) & 1u]), ((t - 1u) >> 1) & 1u, abort_flag));
          if (!ok) {
            if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 800);
            *abort_flag = 1;
            break;
          }
          tcgen05_fence_after();
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            uint32_t acc[32];
            tmem_ld_32x32b_x32(t_o + c * 32, acc);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
            tmem_st_32x32b_x32(t_o + c * 32, acc);
          }
          tmem_st_wait();
        }
        // ---- P = exp2(S * scale - max) as bf16 into tensor memory: row = lane, two values per
        //      32-bit column, which is the form tcgen05.mma reads an A operand from TMEM in
        const float neg_m = -m_run;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t w[32];
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const float a = pf_exp2(fmaf(__uint_as_float(v[2 * c]), scale, neg_m));
          const float b = pf_exp2(fmaf(__uint_as_float(v[2 * c + 1]), scale, neg_m));
          sum0 += a;
          sum1 += b;
          w[c] = pack_bf16(a, b);
        }
        tmem_st_32x32b_x32(t_p + (t & 1u) * 64, w);
        l_run = l_run * alpha + (sum0 + sum1);
        tmem_st_wait();
        tcgen05_fence_before();     // TMEM reads and writes above are ordered before the next MMAs
        mbar_arrive(smem_u32(&p_full[t & 1u]));
        ++step_total;
      }
      if (ok) {
        // The last PV of the item.
        const uint32_t last = step_total - 1u;
        ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_full[last & 1u]), (last >> 1) & 1u, abort_flag));
        if (!ok) {
          if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 600);
          *abort_flag = 1;
        }
      }
      // Row sum = the two threads' partial sums, added in a fixed order. The barrier is taken on
      // every path so that a pair never splits.
      float* slot = xchg + (step_total & 1u) * 256;
      slot[half * 128 + row] = l_run;
      named_bar_sync(pair_barrier, 64);
      if (ok) {
        tcgen05_fence_after();
        const float inv = 1.f / (slot[row] + slot[128 + row]);
        __nv_bfloat16* dst = pp.out + (static_cast<size_t>(it.q_tok0 + row) * p.q_heads + it.head) * 128 + half * 64;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t acc[32];
          tmem_ld_32x32b_x32(t_o + c * 32, acc);
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
    }
  } else if (warp == 8 || warp == 10 || warp == 11) {
    // ---------------------------------------------------------------- TMA producers (K ring, V ring)
    // Boxes: with pages of 8 tokens or more, one box is an 8-token group with both halves of the
    // row (2 KiB); smaller pages fill the two atoms of a group row by row, one box per page and atom.
    const bool is_v = warp == 10;
    const CUtensorMap* tmap = is_v ? &tmap_v : &tmap_k;
    uint8_t* ring = is_v ? v_smem : k_smem;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    // The tensor-memory engine takes of the order of a hundred cycles per copy instruction, so the
    // number of boxes per tile matters. K tiles need a uniform 8-token group stride (the 128 tokens
    // are the N extent of one MMA), which caps a box at one group. A V tile is consumed 16 tokens per
    // MMA, so with pages of 16 tokens or more one box is 16 tokens: [lo g0 | lo g1 | hi g0 | hi g1].
    const bool v_pages = is_v && p.page_size >= 16;
    const int tb = v_pages ? 16 : min(p.page_size, 8);
    const int log2_tb = v_pages ? 4 : min(p.log2_ps, 3);
    // Issuing a copy costs the issuing warp about 70 cycles per box, so the 16 boxes of a K tile are
    // split between warps 8 and 11 (each arrives with half the tile's bytes).
    const int parts = is_v ? 1 : 2;
    const int part = warp == 11 ? 1 : 0;
    const int boxes = (kPfTileKv >> log2_tb) / parts;  // boxes this warp issues per tile
    const int first_box = part * boxes;
    const int reps = (boxes + 31) >> 5;
    const bool wide = p.page_size >= 8;
    for (uint32_t iter = 0; next_item(iter, it); ++iter) {
      if (warp == 8) {
        if (lane == 0) {
          mbar_arrive_expect_tx(smem_u32(q_full), kPfQBytes);
          for (int half = 0; half < 2; ++half)
            tma_load_2d(smem_u32(q_smem + half * (kPfQBytes / 2)), &tmap_q, smem_u32(q_full), it.head * 128 + half * 64,
                        it.q_tok0);
        }
        __syncwarp();
      }
      const int head = p.fused ? 2 * it.kvh + (is_v ? 1 : 0) : it.kvh;
      // Page ids are read 128 table slots at a time (four per lane) and the next 128 are requested
      // while the current ones are in use, so no tile waits for a table read of its own.
      const int pages_needed = (it.kv_needed + p.page_size - 1) >> p.log2_ps;
      const long long table_base = it.table_base;
      const long long table_end = p.table_layout == CAKE_RPA_TABLE_2D ? table_base + p.max_pages_per_seq
                                                                      : static_cast<long long>(p.table_len);
      auto load_window = [&](int base_slot, int (&w)[4]) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
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
      int win_cur[4], win_nxt[4];
      load_window(0, win_cur);
      load_window(128, win_nxt);
      bool alive = true;
      for (int j = 0; j < it.n_steps && alive; ++j) {
        const uint32_t t = step_total;
        const uint32_t slot = t % kPfRing;
        const uint32_t parity = (t / kPfRing) & 1u;
        const int first_slot = (j * kPfTileKv) >> p.log2_ps;
        if (first_slot >= win_base + 128) {  // a tile never straddles two windows
          win_base += 128;
#pragma unroll
          for (int r = 0; r < 4; ++r) win_cur[r] = win_nxt[r];
          load_window(win_base + 128, win_nxt);
        }
        {
          alive = __all_sync(0xffffffffu, pf_wait(smem_u32(&empty[slot]), parity ^ 1u, abort_flag));
        }
        if (!alive) {
          if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, (is_v ? 150 : 100) + j);
          *abort_flag = 1;
          break;
        }
        const uint32_t bar = smem_u32(&full[slot]);
        if (lane == 0) mbar_arrive_expect_tx(bar, kPfTileBytes / parts);
        __syncwarp();
        const uint32_t sbase = smem_u32(ring + slot * kPfTileBytes);
        for (int rep = 0; rep < reps; ++rep) {
          const int b = lane + rep * 32;
          const int tok_in_tile = (first_box + b) * tb;
          const int tok = j * kPfTileKv + tok_in_tile;
          const int rel = (tok >> p.log2_ps) - win_base;  // 0..127 for the boxes of this tile
          const int src = rel & 31;
          const int w0 = __shfl_sync(0xffffffffu, win_cur[0], src);
          const int w1 = __shfl_sync(0xffffffffu, win_cur[1], src);
          const int w2 = __shfl_sync(0xffffffffu, win_cur[2], src);
          const int w3 = __shfl_sync(0xffffffffu, win_cur[3], src);
          if (b < boxes) {
            const int which = (rel >> 5) & 3;
            const int from = which == 0 ? w0 : which == 1 ? w1 : which == 2 ? w2 : w3;
            const int page = tok < it.kv_needed ? from : p.total_pages;
            const int off = tok & (p.page_size - 1);
            const uint32_t gbase = sbase + static_cast<uint32_t>((tok_in_tile >> 3) * kPfGroupBytes);  // 16 tokens = 4 KiB too
            if (wide) {
              tma_load_5d(gbase, tmap, bar, 0, off, 0, head, page);
            } else {
              const uint32_t dst = gbase + static_cast<uint32_t>((tok_in_tile & 7) * 128);
              tma_load_5d(dst, tmap, bar, 0, off, 0, head, page);
              tma_load_5d(dst + 1024, tmap, bar, 0, off, 1, head, page);
            }
          }
        }
        __syncwarp();
        ++loads_issued;
        ++step_total;
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    constexpr uint32_t idesc = umma_idesc_bf16_f32(kPfTileQ, 128, 0, 0);     // S = Q K^T, both K-major
    constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(kPfTileQ, 128, 0, 1);  // O += P V, V MN-major
    // Shared-memory descriptors, split into the low word (address field, which changes per MMA, and
    // the leading offset) and the high word (stride offset, version, swizzle mode).
    //   Q:       K-major, 8-row groups 1 KiB apart; the second 64 elements of a row 16 KiB further.
    //   K tile:  K-major, 8-token groups 2 KiB apart; the second 64 elements of a row are the next atom.
    //   V tile:  [token][d] MN-major: the two 64-wide halves 1 KiB apart (leading offset), 8-token
    //            groups 2 KiB apart (stride offset); a K step of 16 tokens is two groups.
    const uint32_t desc_hi_1024 = static_cast<uint32_t>(umma_desc_sw128(0, 16, 1024) >> 32);
    const uint32_t desc_hi_kv = static_cast<uint32_t>(umma_desc_sw128(0, 16, kPfGroupBytes) >> 32);
    const uint32_t desc_q_lo = static_cast<uint32_t>(umma_desc_sw128(smem_u32(q_smem), 16, 1024));
    const uint32_t desc_k_lo = static_cast<uint32_t>(umma_desc_sw128(smem_u32(k_smem), 16, kPfGroupBytes));
    // V with 16-token boxes: halves 2 KiB apart, the two 8-token groups of a box 1 KiB apart.
    const bool v_pages = p.page_size >= 16;
    const uint32_t desc_v_lo = static_cast<uint32_t>(umma_desc_sw128(smem_u32(v_smem), v_pages ? 2048 : 1024, kPfGroupBytes));
    const uint32_t desc_hi_v = v_pages ? desc_hi_1024 : desc_hi_kv;
    for (uint32_t iter = 0; next_item(iter, it); ++iter) {
      int where = 200;
      auto issue_qk = [&](uint32_t t) {
        const uint32_t k_lo = desc_k_lo + (t % kPfRing) * (kPfTileBytes >> 4);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t a_lo = desc_q_lo + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
          const uint32_t b_lo = k_lo + (((ks >> 2) * 1024 + (ks & 3) * 32) >> 4);
          tcgen05_mma_bf16(tmem_base, pf_desc(a_lo, desc_hi_1024), pf_desc(b_lo, desc_hi_kv), idesc, ks != 0 ? 1u : 0u);
        }
        tcgen05_commit(smem_u32(s_full));
        tcgen05_commit(smem_u32(&k_empty[t % kPfRing]));
      };
      auto wait_tile = [&](uint64_t* full, uint32_t t) -> bool {
        const bool arrived = __all_sync(0xffffffffu, pf_wait(smem_u32(&full[t % kPfRing]), (t / kPfRing) & 1u, abort_flag));
        return arrived;
      };
      // S = Q K^T runs two steps ahead of O += P V: S(t+2) is issued as soon as the softmax warps
      // have taken S(t+1) into registers, which is right after they finish step t, and before PV(t);
      // the softmax never waits for a score tile, and PV(t) still finishes well inside step t+1.
      auto next_scores = [&](uint32_t t_next, uint32_t t_consumed) -> bool {
        where = 300;
        if (!wait_tile(k_full, t_next)) return false;
        where = 350;
        {
          const bool taken = __all_sync(0xffffffffu, pf_wait(smem_u32(s_free), t_consumed & 1u, abort_flag));
          if (!taken) return false;
        }
        tcgen05_fence_after();
        {
          if (lane == 0) issue_qk(t_next);
        }
        __syncwarp();
        return true;
      };
      bool ok = __all_sync(0xffffffffu, pf_wait(smem_u32(q_full), iter & 1u, abort_flag));
      if (ok) ok = wait_tile(k_full, step_total);
      if (ok) {
        tcgen05_fence_after();
        if (lane == 0) issue_qk(step_total);
        __syncwarp();
        if (it.n_steps > 1) ok = next_scores(step_total + 1, step_total);
        for (int j = 0; j < it.n_steps && ok; ++j) {
          const uint32_t t = step_total;
          where = 380;
          ok = wait_tile(v_full, t);
          if (!ok) break;
          // V rows at or beyond kv_len are zeroed (page tails may hold anything; 0 * NaN would
          // poison the product) before the tensor core reads them.
          const int first_bad = max(it.kv_len - j * kPfTileKv, 0);
          if (first_bad < kPfTileKv) {
            uint8_t* v_base = v_smem + (t % kPfRing) * kPfTileBytes;
            for (int e = lane; e < (kPfTileKv - first_bad) * 16; e += 32) {
              const int vrow = first_bad + (e >> 4);
              const int piece = e & 15;
              const int at = v_pages ? (vrow >> 4) * 4096 + (piece >> 3) * 2048 + ((vrow >> 3) & 1) * 1024
                                     : (vrow >> 3) * kPfGroupBytes + (piece >> 3) * 1024;
              *reinterpret_cast<uint4*>(v_base + at + (vrow & 7) * 128 + (piece & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async_smem();
            __syncwarp();
          }
          where = 400;
          {
            ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&p_full[t & 1u]), (t >> 1) & 1u, abort_flag));
          }
          if (!ok) break;
          if (j + 2 < it.n_steps) {
            ok = next_scores(t + 2, t + 1);
            if (!ok) break;
          }
          tcgen05_fence_after();
          if (lane == 0) {
            const uint32_t a_base = tmem_base + kPfTmemP + (t & 1u) * 64;  // 8 columns per 16-token K step
            const uint32_t b_base = desc_v_lo + (t % kPfRing) * (kPfTileBytes >> 4);
            tcgen05_mma_bf16_ts(tmem_base + 128, a_base, pf_desc(b_base, desc_hi_v), idesc_pv, j != 0 ? 1u : 0u);
#pragma unroll
            for (int ks = 1; ks < 8; ++ks)
              tcgen05_mma_bf16_ts(tmem_base + 128, a_base + ks * 8, pf_desc(b_base + ((ks * 2 * kPfGroupBytes) >> 4), desc_hi_v),
                                  idesc_pv, 1u);
            tcgen05_commit(smem_u32(&pv_full[t & 1u]));
            tcgen05_commit(smem_u32(&v_empty[t % kPfRing]));
          }
          __syncwarp();
          ++step_total;
        }
      }
      if (!ok) {
        if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, where);
        *abort_flag = 1;
      }
      __syncwarp();
    }
  }

  // ---- orderly exit
  __syncthreads();
  if (*abort_flag) {
    if ((warp == 8 || warp == 10 || warp == 11) && lane == 0) {
      // loads already issued must land before shared memory is released
      uint64_t* full = warp == 10 ? v_full : k_full;
      for (uint32_t back = 0; back < kPfRing && back < loads_issued; ++back) {
        const uint32_t t = step_total - 1 - back;
        mbar_wait_bounded(smem_u32(&full[t % kPfRing]), (t / kPfRing) & 1u, 200000000ll);
      }
      if (warp == 8) mbar_wait_bounded(smem_u32(q_full), 0, 1000000ll);
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
