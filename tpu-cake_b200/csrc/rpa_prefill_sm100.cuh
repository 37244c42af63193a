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
//       warp 8           TMA producer: query tiles, then 64-token K/V stages gathered page by page
//                        (four boxes per page: K lo/hi, V lo/hi halves of the 128-wide row, so that a
//                        stage is laid out [half][token][128 B] as tcgen05 operands need; no multicast)
//       warp 9           tcgen05.mma issuer: S = Q K^T (128x64, K-major operands) and PV = P V
//                        (128x128, V consumed in place as an MN-major operand) into TMEM
//     S is read from TMEM with tcgen05.ld (a thread owns a row, so the row maximum and sum need no
//     shuffles), P goes back through shared memory in the 128-byte-swizzled K-major layout, the
//     running output stays in registers in f32 and is rescaled as the maximum moves.
#pragma once

namespace cake {

constexpr int kPfThreads = 384;
constexpr int kPfTileQ = 128;
constexpr int kPfTileKv = 64;
constexpr int kPfStages = 3;
constexpr int kPfQBytes = kPfTileQ * 256;        // one sub-tile of queries: [2 halves][128 rows][128 B]
constexpr int kPfStageBytes = kPfTileKv * 512;   // K [2][64][128 B] then V [2][64][128 B]
constexpr int kPfPBytes = kPfTileQ * 128;        // P sub-tile: [128 rows][64 bf16]
constexpr int kPfSmemBytes = 2 * kPfQBytes + kPfStages * kPfStageBytes + 2 * kPfPBytes + 1024 + 1024;
constexpr uint32_t kPfTmemCols = 512;            // S0 @0, S1 @64, PV0 @128, PV1 @256
constexpr long long kPfBarrierBudget = 2000000000ll;

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
  uint8_t* kv_smem = q_smem + 2 * kPfQBytes;                  // [stages][K 16 KiB | V 16 KiB]
  uint8_t* p_smem = kv_smem + kPfStages * kPfStageBytes;      // [2 sub-tiles][128][128 B]
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_smem + 2 * kPfPBytes);
  uint64_t* q_full = bars;              // [1]
  uint64_t* kv_full = bars + 1;         // [stages]
  uint64_t* kv_empty = kv_full + kPfStages;
  uint64_t* s_full = kv_empty + kPfStages;  // [2]
  uint64_t* p_full = s_full + 2;            // [2]
  uint64_t* pv_full = p_full + 2;           // [2]
  uint64_t* drain_bar = pv_full + 2;        // [1]
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
      mbar_init(smem_u32(&p_full[g]), 128);
      mbar_init(smem_u32(&pv_full[g]), 1);
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
      uint8_t* p_row = p_smem + g * kPfPBytes + row * 128;
      for (uint32_t iter = 0; next_item(iter, it); ++iter) {
        const int limit = min(it.prior + it.q0 + row, it.kv_len - 1);  // last position this row sees
        float o[128];
#pragma unroll
        for (int i = 0; i < 128; ++i) o[i] = 0.f;
        float m_run = kNegBig, l_run = 0.f;
        bool ok = true;
        for (int j = 0; j < it.n_steps; ++j) {
          ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&s_full[g]), step_total & 1u, abort_flag));
          if (!ok) {
            if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 500 + g);
            *abort_flag = 1;
            break;
          }
          tcgen05_fence_after();
          const int pos0 = j * kPfTileKv;
          const bool need_mask = pos0 + kPfTileKv - 1 > limit;
          // ---- pass 1: row maximum of the scaled, masked scores
          float mx = m_run;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_s + half * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) {
              float sv = __uint_as_float(v[c]) * p.scale_log2;
              if (need_mask && pos0 + half * 32 + c > limit) sv = kNegBig;
              mx = fmaxf(mx, sv);
            }
          }
          const float alpha = exp2f(m_run - mx);
          m_run = mx;
          // ---- pass 2: P = exp2(S - max) as bf16 into shared memory (K-major, 128-byte swizzle)
          float sum = 0.f;
#pragma unroll
          for (int half = 0; half < 2; ++half) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_s + half * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int c = c4 * 8 + e * 2;
                float a = exp2f(__uint_as_float(v[c]) * p.scale_log2 - mx);
                float b = exp2f(__uint_as_float(v[c + 1]) * p.scale_log2 - mx);
                if (need_mask) {
                  if (pos0 + half * 32 + c > limit) a = 0.f;
                  if (pos0 + half * 32 + c + 1 > limit) b = 0.f;
                }
                // The sum uses the rounded weights, the values the tensor core multiplies with.
                const __nv_bfloat162 pk = __floats2bfloat162_rn(a, b);
                sum += __low2float(pk) + __high2float(pk);
                w[e] = *reinterpret_cast<const uint32_t*>(&pk);
              }
              const int chunk = half * 4 + c4;
              *reinterpret_cast<uint4*>(p_row + ((chunk ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
          l_run = l_run * alpha + sum;
          fence_proxy_async_smem();   // P written through the generic proxy, read by the tensor core
          tcgen05_fence_before();     // the S reads above are ordered before the MMA that overwrites S
          mbar_arrive(smem_u32(&p_full[g]));
          // ---- O = O * alpha + P V
          ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_full[g]), step_total & 1u, abort_flag));
          if (!ok) {
            if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, 600 + g);
            *abort_flag = 1;
            break;
          }
          tcgen05_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld_32x32b_x32(t_pv + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) o[c * 32 + e] = o[c * 32 + e] * alpha + __uint_as_float(v[e]);
          }
          tcgen05_fence_before();
          ++step_total;
        }
        if (ok && row < it.rows) {
          const float inv = 1.f / l_run;
          __nv_bfloat16* dst = pp.out + (static_cast<size_t>(it.q_tok0 + row) * p.q_heads + it.head0 + g) * 128;
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            uint4 piece;
            piece.x = pack_bf16(o[c * 8 + 0] * inv, o[c * 8 + 1] * inv);
            piece.y = pack_bf16(o[c * 8 + 2] * inv, o[c * 8 + 3] * inv);
            piece.z = pack_bf16(o[c * 8 + 4] * inv, o[c * 8 + 5] * inv);
            piece.w = pack_bf16(o[c * 8 + 6] * inv, o[c * 8 + 7] * inv);
            *reinterpret_cast<uint4*>(dst + c * 8) = piece;
          }
        }
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
      const int tb = p.box_tokens;
      const int boxes = kPfTileKv >> p.log2_box;
      for (uint32_t iter = 0; next_item(iter, it); ++iter) {
        if (lane == 0) {
          mbar_arrive_expect_tx(smem_u32(q_full), static_cast<uint32_t>(sub * kPfQBytes));
          for (int g = 0; g < sub; ++g)
            for (int half = 0; half < 2; ++half)
              tma_load_2d(smem_u32(q_smem + g * kPfQBytes + half * (kPfQBytes / 2)), &tmap_q, smem_u32(q_full),
                          (it.head0 + g) * 128 + half * 64, it.q_tok0);
          ++q_issued;
        }
        __syncwarp();
        for (int j = 0; j < it.n_steps; ++j) {
          const uint32_t stage = kv_pos % kPfStages;
          const uint32_t parity = (kv_pos / kPfStages) & 1u;
          // Page ids of this stage's boxes first, so the table read overlaps the wait for the slot.
          int my_page[2] = {p.total_pages, p.total_pages};  // out-of-range coordinate: zero fill
          int my_off[2] = {0, 0};
#pragma unroll
          for (int rep = 0; rep < 2; ++rep) {
            const int b = lane + rep * 32;
            const int tok = j * kPfTileKv + b * tb;
            if (b < boxes && tok < it.kv_needed) {
              const int page_slot = tok >> p.log2_ps;
              int page = rpa_page_lookup(p, it.seq, page_slot);
              if (page < 0 || page >= p.total_pages) {
                rpa_record(p.status, 3, it.seq, page_slot, page);
                page = p.total_pages;
              }
              my_page[rep] = page;
              my_off[rep] = tok & (p.page_size - 1);
            }
          }
          if (!__all_sync(0xffffffffu, pf_wait(smem_u32(&kv_empty[stage]), parity ^ 1u, abort_flag))) {
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
              const uint32_t dst = sbase + static_cast<uint32_t>(b * tb * 128);
              tma_load_5d(dst, &tmap_k, bar, 0, my_off[rep], 0, hk, my_page[rep]);
              tma_load_5d(dst + 8192, &tmap_k, bar, 0, my_off[rep], 1, hk, my_page[rep]);
              tma_load_5d(dst + 16384, &tmap_v, bar, 0, my_off[rep], 0, hv, my_page[rep]);
              tma_load_5d(dst + 24576, &tmap_v, bar, 0, my_off[rep], 1, hv, my_page[rep]);
            }
          }
          __syncwarp();
          ++kv_pos;
        }
      }
    } else if (warp == 9) {
      // ---------------------------------------------------------------- MMA issuer
      constexpr uint32_t idesc_qk = umma_idesc_bf16_f32(kPfTileQ, kPfTileKv, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16_f32(kPfTileQ, 128, 0, 1);
      for (uint32_t iter = 0; next_item(iter, it); ++iter) {
        int where = 200;
        // Waits for stage `pos`, then zeroes its V rows at or beyond kv_len (page tails may hold
        // anything; 0 * NaN would poison the product) before the tensor core reads them.
        auto stage_ready = [&](uint32_t pos, int j) -> bool {
          if (!__all_sync(0xffffffffu, pf_wait(smem_u32(&kv_full[pos % kPfStages]), (pos / kPfStages) & 1u, abort_flag)))
            return false;
          const int first_bad = max(it.kv_len - j * kPfTileKv, 0);
          if (first_bad < kPfTileKv) {
            uint8_t* v_base = kv_smem + (pos % kPfStages) * kPfStageBytes + 16384;
            for (int e = lane; e < (kPfTileKv - first_bad) * 16; e += 32) {
              const int row = first_bad + (e >> 4);
              const int piece = e & 15;
              *reinterpret_cast<uint4*>(v_base + (piece >> 3) * 8192 + row * 128 + (piece & 7) * 16) = make_uint4(0u, 0u, 0u, 0u);
            }
            fence_proxy_async_smem();
          }
          __syncwarp();
          return true;
        };
        auto issue_qk = [&](int g, uint32_t pos) {
          const uint32_t qa = smem_u32(q_smem + g * kPfQBytes);
          const uint32_t kb = smem_u32(kv_smem + (pos % kPfStages) * kPfStageBytes);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t a_desc = umma_desc_sw128(qa + (ks >> 2) * 16384 + (ks & 3) * 32, 16, 1024);
            const uint64_t b_desc = umma_desc_sw128(kb + (ks >> 2) * 8192 + (ks & 3) * 32, 16, 1024);
            tcgen05_mma_bf16(tmem_base + g * 64, a_desc, b_desc, idesc_qk, ks != 0 ? 1u : 0u);
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
            for (int g = 0; g < sub; ++g) {
              where = 400 + g;
              ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&p_full[g]), step_total & 1u, abort_flag));
              if (!ok) break;
              tcgen05_fence_after();
              if (lane == 0) {
                const uint32_t pa = smem_u32(p_smem + g * kPfPBytes);
                const uint32_t vb = smem_u32(kv_smem + (kv_pos % kPfStages) * kPfStageBytes + 16384);
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
                  const uint64_t a_desc = umma_desc_sw128(pa + ks * 32, 16, 1024);
                  const uint64_t b_desc = umma_desc_sw128(vb + ks * 2048, 8192, 1024);
                  tcgen05_mma_bf16(tmem_base + 128 + g * 128, a_desc, b_desc, idesc_pv, ks != 0 ? 1u : 0u);
                }
                tcgen05_commit(smem_u32(&pv_full[g]));
                if (j + 1 < it.n_steps) issue_qk(g, kv_pos + 1);
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
