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
//   cake_rpa_prefill_sm100         persistent, one CTA per SM. A work item is 128 query tokens of TWO
//                                  query heads of one KV group (tiles A and B), walked over the KV
//                                  range in steps of 128 tokens: every K and V tile is loaded once for
//                                  both heads, and while the softmax of one tile runs the tensor core
//                                  works for the other, so neither waits for the other's latency.
//                                  (An odd group size pairs nothing: tile B is then left out.)
//       warps 0-3   softmax of tile A, warps 4-7 softmax of tile B: one thread per query row (= TMEM
//                   lane), so a row's maximum and sum need no exchange. A step brings its whole score
//                   row (128 columns) into registers with one wait, forms P = exp2(S * scale - max)
//                   and writes it back into tensor memory as packed bf16 OVER the columns of S (the
//                   tensor core reads it from there as the A operand of O += P V). The output row
//                   accumulates in TMEM over all steps and is read, rescaled and written back only
//                   when its maximum has moved by more than 2^8.
//       warps 8, 11 TMA producers of the two query tiles and of the K ring, half a tile each
//       warp 10     TMA producer of the V ring. K tiles are gathered page by page in boxes of one
//                   8-token group (both 64-element halves of the row: 2 KiB), laid out
//                   [group][lo | hi][8 rows][128 B]: groups a uniform 2 KiB apart, which is what the
//                   tcgen05 shared-memory descriptor of a 128-token operand needs. V tiles are read
//                   16 tokens per MMA, so their boxes are 16 tokens (4 KiB) when pages allow.
//                   Never multicast.
//       warp 9      tcgen05.mma issuer, in the order S_A(0) S_B(0) | O_A+=P_A V(j), S_A(j+1),
//                   O_B+=P_B V(j), S_B(j+1) | ...: the tensor pipe executes in issue order, so the
//                   next S of a tile follows the P V that read the P it overwrites.
//     TMEM: S_A columns 0-127 (P_A over 0-63), S_B 128-255 (P_B over 128-191), O_A 256-383, O_B 384-511.
#pragma once

namespace cake {

constexpr int kPfThreads = 384;
constexpr int kPfTileQ = 128;                    // query rows per tile (one query head)
constexpr int kPfTileKv = 128;                   // KV tokens per step
constexpr int kPfRingK = 2;                      // slots of the K ring (a third slot measured no faster)
constexpr int kPfRingV = 2;                      // slots of the V ring
constexpr int kPfQBytes = kPfTileQ * 256;        // one query tile: [2 halves][128 rows][128 B]
constexpr int kPfTileBytes = kPfTileKv * 256;    // a K or V tile: [16 groups][lo | hi][8 rows][128 B]
constexpr int kPfGroupBytes = 2048;              // one 8-token group of a K or V tile
constexpr int kPfTailBytes = 1024;               // barriers, TMEM slot, item slots
constexpr int kPfSmemBytes = 2 * kPfQBytes + (kPfRingK + kPfRingV) * kPfTileBytes + kPfTailBytes;
constexpr uint32_t kPfTmemCols = 512;
constexpr uint32_t kPfTmemO = 256;               // first column of O_A; tile X: S at 128 X, O at 256 + 128 X
constexpr long long kPfBarrierBudget = 2000000000ll;
constexpr float kPfRescale = 8.f;                // log2 units the row maximum may lag before O is rescaled

struct PrefillParams {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int32_t* kv_lens;
  const int32_t* cu_q_lens;
  int32_t first_seq;       // sequences [first_seq, num_seqs) are handled here
  int32_t heads_items;     // work items per (sequence, query tile): one per query head, or per pair of heads
  int32_t paired;          // 1: an item is heads 2i and 2i+1 of one KV group (group size even)
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

// Two float32 values in one 64-bit register, for the packed (two per instruction) arithmetic of sm_100.
__device__ __forceinline__ uint64_t pf_pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ void pf_unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}

__device__ __forceinline__ uint64_t pf_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

__device__ __forceinline__ uint64_t pf_add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ float pf_max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Warp-collective: lane i writes 16 consecutive 32-bit columns of TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// Warp-collective: lane i receives 16 consecutive f32 columns of TMEM lane (base lane + i).
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

__global__ void __launch_bounds__(kPfThreads, 1)
    cake_rpa_prefill_sm100(const __grid_constant__ CUtensorMap tmap_q,
                           const __grid_constant__ CUtensorMap tmap_k,
                           const __grid_constant__ CUtensorMap tmap_v, const PrefillParams pp) {
  const RpaParams& p = pp.r;
  // The tiles need 1 KiB alignment (128-byte swizzle atoms): requested and checked.
  extern __shared__ __align__(1024) uint8_t pf_smem_raw[];
  uint8_t* smem = pf_smem_raw;
  if (smem_u32(smem) & 1023u) {
    if (threadIdx.x == 0) rpa_record(p.status, 5, blockIdx.x, static_cast<int>(smem_u32(smem) & 1023u), 0);
    return;
  }
  uint8_t* q_smem = smem;                                  // [tile A | tile B][2 halves][128 rows][128 B]
  uint8_t* k_smem = q_smem + 2 * kPfQBytes;                // [ring][16 groups][lo | hi][8 rows][128 B]
  uint8_t* v_smem = k_smem + kPfRingK * kPfTileBytes;      // same
  uint64_t* bars = reinterpret_cast<uint64_t*>(v_smem + kPfRingV * kPfTileBytes);
  uint64_t* q_full = bars;                 // [1]
  uint64_t* k_full = bars + 1;             // [K ring]
  uint64_t* k_empty = k_full + kPfRingK;   // [K ring]
  uint64_t* v_full = k_empty + kPfRingK;   // [V ring]
  uint64_t* v_empty = v_full + kPfRingV;   // [V ring]
  uint64_t* s_full = v_empty + kPfRingV;   // [2 tiles] S = Q K^T of the tile's current step is complete
  uint64_t* p_full = s_full + 2;           // [2 tiles][2 halves] 128 rows x 64 KV tokens of P are in tensor memory
  uint64_t* pv_done = p_full + 4;          // [2 tiles] O += P V of the tile's current step is complete
  uint64_t* drain_bar = pv_done + 2;       // [1]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(drain_bar + 1);
  volatile uint32_t* abort_flag = tmem_base_slot + 1;
  volatile int32_t* item_slot = reinterpret_cast<volatile int32_t*>(tmem_base_slot + 2);  // [2]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(q_full), 1);
    for (int s = 0; s < kPfRingK; ++s) {
      mbar_init(smem_u32(&k_full[s]), 2);  // two producer warps, half a tile each
      mbar_init(smem_u32(&k_empty[s]), 1);
    }
    for (int s = 0; s < kPfRingV; ++s) {
      mbar_init(smem_u32(&v_full[s]), 1);
      mbar_init(smem_u32(&v_empty[s]), 1);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(smem_u32(&s_full[x]), 1);
      mbar_init(smem_u32(&p_full[2 * x]), 128);
      mbar_init(smem_u32(&p_full[2 * x + 1]), 128);
      mbar_init(smem_u32(&pv_done[x]), 1);
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

  // Running counts that persist across work items; every role advances them the same way.
  // kv_total numbers the K / V tiles (ring slot kv_total % ring, phase (kv_total / ring) & 1, per ring);
  // tile_total[x] numbers the steps tile x has taken (phase of its three barriers: tile_total & 1).
  uint32_t kv_total = 0;
  uint32_t tile_total[2] = {0u, 0u};
  uint32_t loads_issued = 0;  // producers: tiles issued, for the orderly exit

  struct Item {
    int id, seq, q0, kv_len, head, kvh, two, prior, rows, kv_needed, n_steps, q_tok0, table_base;
  };
  // Hands the next work item to the whole CTA. One thread claims (an item, or -1 after an abort),
  // one item ahead, so that every thread leaves its loop in the same iteration. The barrier also
  // separates items: when it opens, every role has finished the previous one, so the query buffers
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
    it.two = pp.paired;
    it.head = (id % pp.heads_items) * (pp.paired ? 2 : 1);  // tile A's query head; tile B's is the next one
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
    // Warps 0-3 own tile A, warps 4-7 tile B; thread = query row = TMEM lane 32 (warp & 3) + lane.
    const int x = warp >> 2;
    const int row = (warp & 3) * 32 + lane;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    const uint32_t t_s = t_lane + x * 128;             // S of this tile; P is written over its first 64 columns
    const uint32_t t_o = t_lane + kPfTmemO + x * 128;  // O of this tile
    const float scale = p.scale_log2;  // positive: checked on the host
    for (uint32_t iter = 0; next_item(iter, it); ++iter) {
      if (x == 1 && !it.two) continue;  // nothing is paired with tile A in this batch
      const int limit = min(it.prior + it.q0 + row, it.kv_len - 1);  // last position this row sees
      // Running maximum (log2 domain, scaled) and sum of the row. The maximum is allowed to lag by
      // kPfRescale, so the exponentials are bounded by 2^kPfRescale.
      float m_run = kNegBig, l_run = 0.f;
      bool ok = true;
      int where = 500;
      for (int j = 0; j < it.n_steps; ++j) {
        const uint32_t t = tile_total[x];
        ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&s_full[x]), t & 1u, abort_flag));
        if (!ok) break;
        tcgen05_fence_after();
        const int pos0 = j * kPfTileKv;
        // The whole score row comes into registers with one wait: four loads in flight together
        // (a load's round trip through tensor memory is several hundred cycles, and a step that
        // waited for eight of them in turn spent most of its time there).
        uint32_t v[128];
        tmem_ld_32x32b_x32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        tmem_ld_32x32b_x32(t_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        tmem_ld_32x32b_x32(t_s + 64, *reinterpret_cast<uint32_t(*)[32]>(&v[64]));
        tmem_ld_32x32b_x32(t_s + 96, *reinterpret_cast<uint32_t(*)[32]>(&v[96]));
        tmem_ld_wait();
        // Only the steps that cross the row's causal limit (or the end of the sequence) mask.
        if (__any_sync(0xffffffffu, pos0 + kPfTileKv - 1 > limit)) {
#pragma unroll
          for (int c = 0; c < 128; ++c)
            if (pos0 + c > limit) v[c] = 0xff800000u;  // -inf
        }
        float mr0 = __uint_as_float(v[0]), mr1 = __uint_as_float(v[1]), mr2 = __uint_as_float(v[2]), mr3 = __uint_as_float(v[3]);
#pragma unroll
        for (int c = 4; c < 128; c += 8) {
          mr0 = pf_max3(mr0, __uint_as_float(v[c]), __uint_as_float(v[c + 1]));
          mr1 = pf_max3(mr1, __uint_as_float(v[c + 2]), __uint_as_float(v[c + 3]));
          if (c + 4 < 128) {
            mr2 = pf_max3(mr2, __uint_as_float(v[c + 4]), __uint_as_float(v[c + 5]));
            mr3 = pf_max3(mr3, __uint_as_float(v[c + 6]), __uint_as_float(v[c + 7]));
          }
        }
        const float mx = fmaxf(fmaxf(mr0, mr1), fmaxf(mr2, mr3)) * scale;
        float alpha = 1.f;
        if (mx > m_run + kPfRescale) {
          alpha = pf_exp2(m_run - mx);
          m_run = mx;
        }
        // Rare: the accumulator is read and rewritten once the previous O += P V of this tile is
        // complete; the next one is issued only after p_full below.
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          where = 800;
          ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_done[x]), (t - 1u) & 1u, abort_flag));
          if (!ok) break;
          tcgen05_fence_after();
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t acc[16];
            tmem_ld_32x32b_x16(t_o + c * 16, acc);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 16; ++e) acc[e] = __float_as_uint(__uint_as_float(acc[e]) * alpha);
            tmem_st_32x32b_x16(t_o + c * 16, acc);
          }
          tmem_st_wait();
          where = 500;
        }
        // ---- P = exp2(S * scale - max) as bf16 pairs, written over the columns of S (all of it is
        //      in registers): 32 scores become 16 packed columns. The packing rounds half up with
        //      integer adds and a byte permute, so that only the exponentials use the XU pipe,
        //      which the conversion instruction would otherwise share with them.
        // Scale-and-subtract and the row sum run two values per instruction (packed f32x2), the
        // packing to bf16 is one conversion per pair: the exponentials, on the XU pipe, are the only
        // per-element instructions left. P is announced in two halves of 64 KV tokens, so the
        // tensor core starts O += P V on the first while the second is being formed.
        const uint64_t scale2 = pf_pack2(scale, scale);
        const uint64_t neg_m2 = pf_pack2(-m_run, -m_run);
        uint64_t sum2 = pf_pack2(0.f, 0.f);
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t w[16];
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float x0, x1;
            pf_unpack2(pf_fma2(pf_pack2(__uint_as_float(v[ch * 32 + 2 * c]), __uint_as_float(v[ch * 32 + 2 * c + 1])), scale2, neg_m2), x0, x1);
            const float e0 = pf_exp2(x0);
            const float e1 = pf_exp2(x1);
            sum2 = pf_add2(sum2, pf_pack2(e0, e1));
            // bf16 pair, rounded half up with integer adds and a byte permute (measured faster
            // than the conversion instruction here).
            w[c] = __byte_perm(__float_as_uint(e0) + 0x8000u, __float_as_uint(e1) + 0x8000u, 0x7632);
          }
          tmem_st_32x32b_x16(t_s + ch * 16, w);
          if (ch == 1) {
            tmem_st_wait();
            tcgen05_fence_before();
            mbar_arrive(smem_u32(&p_full[2 * x]));
          }
        }
        float sum0, sum1;
        pf_unpack2(sum2, sum0, sum1);
        l_run = l_run * alpha + (sum0 + sum1);
        tmem_st_wait();
        tcgen05_fence_before();     // TMEM reads and writes above are ordered before the next MMAs
        mbar_arrive(smem_u32(&p_full[2 * x + 1]));
        ++tile_total[x];
      }
      if (ok) {
        // The last O += P V of the item.
        where = 600;
        ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&pv_done[x]), (tile_total[x] - 1u) & 1u, abort_flag));
      }
      if (!ok) {
        if (lane == 0 && !*abort_flag) rpa_record(p.status, 1, blockIdx.x, it.id, where + x);
        *abort_flag = 1;
        continue;
      }
      tcgen05_fence_after();
      const float inv = 1.f / l_run;
      __nv_bfloat16* dst = pp.out + (static_cast<size_t>(it.q_tok0 + row) * p.q_heads + it.head + x) * 128;
      {
        // The whole output row with one wait, as for the scores.
        uint32_t acc[128];
        tmem_ld_32x32b_x32(t_o, *reinterpret_cast<uint32_t(*)[32]>(&acc[0]));
        tmem_ld_32x32b_x32(t_o + 32, *reinterpret_cast<uint32_t(*)[32]>(&acc[32]));
        tmem_ld_32x32b_x32(t_o + 64, *reinterpret_cast<uint32_t(*)[32]>(&acc[64]));
        tmem_ld_32x32b_x32(t_o + 96, *reinterpret_cast<uint32_t(*)[32]>(&acc[96]));
        tmem_ld_wait();
        if (row < it.rows) {
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            uint4 piece;
            piece.x = pack_bf16(__uint_as_float(acc[e * 8 + 0]) * inv, __uint_as_float(acc[e * 8 + 1]) * inv);
            piece.y = pack_bf16(__uint_as_float(acc[e * 8 + 2]) * inv, __uint_as_float(acc[e * 8 + 3]) * inv);
            piece.z = pack_bf16(__uint_as_float(acc[e * 8 + 4]) * inv, __uint_as_float(acc[e * 8 + 5]) * inv);
            piece.w = pack_bf16(__uint_as_float(acc[e * 8 + 6]) * inv, __uint_as_float(acc[e * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + e * 8) = piece;
          }
        }
      }
      tcgen05_fence_before();  // the accumulator reads are ordered before the next item's MMAs
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
    const uint32_t ring_slots = is_v ? kPfRingV : kPfRingK;
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
          mbar_arrive_expect_tx(smem_u32(q_full), it.two ? 2 * kPfQBytes : kPfQBytes);
          for (int x = 0; x < (it.two ? 2 : 1); ++x)
            for (int half = 0; half < 2; ++half)
              tma_load_2d(smem_u32(q_smem + x * kPfQBytes + half * (kPfQBytes / 2)), &tmap_q, smem_u32(q_full),
                          (it.head + x) * 128 + half * 64, it.q_tok0);
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
        const uint32_t t = kv_total;
        const uint32_t slot = t % ring_slots;
        const uint32_t parity = (t / ring_slots) & 1u;
        const int first_slot = (j * kPfTileKv) >> p.log2_ps;
        if (first_slot >= win_base + 128) {  // a tile never straddles two windows
          win_base += 128;
#pragma unroll
          for (int r = 0; r < 4; ++r) win_cur[r] = win_nxt[r];
          load_window(win_base + 128, win_nxt);
        }
        alive = __all_sync(0xffffffffu, pf_wait(smem_u32(&empty[slot]), parity ^ 1u, abort_flag));
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
        ++kv_total;
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
      const int tiles = it.two ? 2 : 1;
      // S_x = Q_x K^T of K tile `t` (one elected lane).
      auto issue_qk = [&](int x, uint32_t t) {
        const uint32_t k_lo = desc_k_lo + (t % kPfRingK) * (kPfTileBytes >> 4);
        const uint32_t q_lo = desc_q_lo + x * (kPfQBytes >> 4);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t a_lo = q_lo + (((ks >> 2) * 16384 + (ks & 3) * 32) >> 4);
          const uint32_t b_lo = k_lo + (((ks >> 2) * 1024 + (ks & 3) * 32) >> 4);
          tcgen05_mma_bf16(tmem_base + x * 128, pf_desc(a_lo, desc_hi_1024), pf_desc(b_lo, desc_hi_kv), idesc, ks != 0 ? 1u : 0u);
        }
        tcgen05_commit(smem_u32(&s_full[x]));
      };
      // One half (64 KV tokens: four 16-token K steps) of O_x += P_x V of V tile `t`; P_x is read
      // from tensor memory, 8 columns per K step.
      auto issue_pv_half = [&](int x, uint32_t t, int half, bool accumulate) {
        const uint32_t a_base = tmem_base + x * 128;
        const uint32_t b_base = desc_v_lo + (t % kPfRingV) * (kPfTileBytes >> 4);
        const uint32_t d = tmem_base + kPfTmemO + x * 128;
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4) {
          const int ks = half * 4 + k4;
          tcgen05_mma_bf16_ts(d, a_base + ks * 8, pf_desc(b_base + ((ks * 2 * kPfGroupBytes) >> 4), desc_hi_v), idesc_pv,
                              (accumulate || ks != 0) ? 1u : 0u);
        }
        if (half == 1) tcgen05_commit(smem_u32(&pv_done[x]));
      };
      auto wait_tile = [&](uint64_t* full, uint32_t t, uint32_t ring_slots) -> bool {
        return __all_sync(0xffffffffu, pf_wait(smem_u32(&full[t % ring_slots]), (t / ring_slots) & 1u, abort_flag));
      };
      bool ok = __all_sync(0xffffffffu, pf_wait(smem_u32(q_full), iter & 1u, abort_flag));
      if (ok) ok = wait_tile(k_full, kv_total, kPfRingK);
      if (ok) {
        tcgen05_fence_after();
        if (lane == 0) {
          for (int x = 0; x < tiles; ++x) issue_qk(x, kv_total);
          tcgen05_commit(smem_u32(&k_empty[kv_total % kPfRingK]));
        }
        __syncwarp();
        for (int j = 0; j < it.n_steps && ok; ++j) {
          const uint32_t t = kv_total;
          const bool more = j + 1 < it.n_steps;
          where = 380;
          ok = wait_tile(v_full, t, kPfRingV);
          if (!ok) break;
          // V rows at or beyond kv_len are zeroed (page tails may hold anything; 0 * NaN would
          // poison the product) before the tensor core reads them.
          const int first_bad = max(it.kv_len - j * kPfTileKv, 0);
          if (first_bad < kPfTileKv) {
            uint8_t* v_base = v_smem + (t % kPfRingV) * kPfTileBytes;
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
          if (more) {
            where = 300;
            ok = wait_tile(k_full, t + 1, kPfRingK);
            if (!ok) break;
          }
          for (int x = 0; x < tiles && ok; ++x) {
            for (int half = 0; half < 2 && ok; ++half) {
              where = 400 + 2 * x + half;
              ok = __all_sync(0xffffffffu, pf_wait(smem_u32(&p_full[2 * x + half]), tile_total[x] & 1u, abort_flag));
              if (!ok) break;
              tcgen05_fence_after();
              if (lane == 0) issue_pv_half(x, t, half, j != 0);
              __syncwarp();
            }
            if (!ok) break;
            if (lane == 0) {
              if (x == tiles - 1) tcgen05_commit(smem_u32(&v_empty[t % kPfRingV]));
              // The next S of this tile overwrites the P that the MMAs above read: issue order
              // is execution order on the tensor pipe.
              if (more) {
                issue_qk(x, t + 1);
                if (x == tiles - 1) tcgen05_commit(smem_u32(&k_empty[(t + 1) % kPfRingK]));
              }
            }
            __syncwarp();
            ++tile_total[x];
          }
          ++kv_total;
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
      const uint32_t ring_slots = warp == 10 ? kPfRingV : kPfRingK;
      for (uint32_t back = 0; back < ring_slots && back < loads_issued; ++back) {
        const uint32_t t = kv_total - 1 - back;
        mbar_wait_bounded(smem_u32(&full[t % ring_slots]), (t / ring_slots) & 1u, 200000000ll);
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
