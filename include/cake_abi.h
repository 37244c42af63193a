/* C ABI of libcake_b200.so: the sm_100a backend for the two kernel targets of tpu-cake's
 * schedule dialect -- the K-sharded BF16 matmul followed by a reduce-scatter, and Inkling
 * ragged paged attention (RPA).
 *
 * Conventions
 *   - Every function returns an int32_t status: 0 = CAKE_OK, negative = error. A textual
 *     description of the last error on the calling thread is returned by cake_last_error().
 *   - The caller owns every device buffer it passes in. The library owns only its handles
 *     and the symmetric receive slots it allocates for the peer-to-peer strategy.
 *   - One process drives one GPU (the current CUDA device at create time). Multi-GPU runs
 *     use one process per GPU; receive slots are shared between processes with CUDA IPC
 *     handles that the host exchanges over its own channel (torch.distributed, MPI, ...).
 *   - Enqueue calls are asynchronous and ordered on the CUDA stream passed in (a
 *     cudaStream_t cast to void*; NULL = the legacy default stream).
 *   - Handles are not thread-safe.
 *   - No function falls back to a CPU implementation.
 */
#ifndef CAKE_ABI_H_
#define CAKE_ABI_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CAKE_OK 0
#define CAKE_ERR_INVALID_ARGUMENT (-1)
#define CAKE_ERR_CUDA (-2)
#define CAKE_ERR_UNSUPPORTED (-3)
#define CAKE_ERR_TIMEOUT (-4)   /* a bounded device-side wait ran out; see cake_status */
#define CAKE_ERR_DEVICE_CHECK (-5) /* a device-side index check failed; see cake_status */
#define CAKE_ERR_STATE (-6)

#define CAKE_MAX_WORLD 8

#define CAKE_DTYPE_F32 0
#define CAKE_DTYPE_BF16 1

/* ---------------------------------------------------------------- general */

/* ABI version of the loaded library. */
int32_t cake_abi_version(void);

/* Last error message of the calling thread (never NULL). */
const char* cake_last_error(void);

/* Device-written status word of the most recent kernels of a handle family.
 * code: 0 = ok, 1 = bounded wait on a shared-memory barrier ran out, 2 = bounded wait on a
 * peer's data or flag ran out, 3 = page index out of range, 4 = sequence metadata out of range,
 * 5 = a kernel found its shared memory misaligned and did nothing.
 * detail0..2 carry coordinates (block, tile / sequence, stage / page slot). */
typedef struct cake_status {
  int32_t code;
  int32_t detail0;
  int32_t detail1;
  int32_t detail2;
} cake_status;

/* ---------------------------------------------------------------- symmetric memory helpers
 * Replaces the remote-DMA scratch the reference allocates inside its Pallas ring kernel
 * (src/tpu_cake/pallas_lowering.py:276-326): receive slots live in ordinary device memory
 * allocated here with cudaMalloc so that they can be exported to peer processes. */
int32_t cake_symm_alloc(size_t bytes, void** out_ptr);           /* zero-filled */
int32_t cake_symm_free(void* ptr);
int32_t cake_ipc_export(void* ptr, uint8_t handle_out[64]);
int32_t cake_ipc_open(const uint8_t handle[64], void** out_ptr);
int32_t cake_ipc_close(void* ptr);

/* ---------------------------------------------------------------- matmul + reduce-scatter
 * Replaces PallasMatmulPlan.build()'s executable (src/tpu_cake/pallas_lowering.py:417-476):
 * the per-device local contraction (_matmul_kernel, :44-50,429-444) followed by the
 * reduce-scatter over the mesh axis (lax.psum_scatter, :459-464, or the Pallas ring, :117-326).
 */

#define CAKE_RS_LOCAL_PARTIAL 0 /* write the partial, laid out owner-major; the host runs the
                                   library collective (NCCL reduce-scatter) on it */
#define CAKE_RS_P2P_OWNER_PUSH 1 /* epilogue pushes each partial tile to its owner GPU; six more
                                    warps of the same kernel sum the W slots in rank order */

typedef struct cake_matmul_rs_desc {
  int64_t m;            /* rows of lhs and of the partial */
  int64_t n;            /* columns of rhs and of the partial */
  int64_t k_local;      /* this rank's share of the contraction dimension */
  int32_t world;        /* mesh size W (1..CAKE_MAX_WORLD) */
  int32_t rank;         /* this process's position on the mesh axis */
  int32_t scatter_dim;  /* 0 = scatter rows (M), 1 = scatter columns (N) */
  int32_t out_dtype;    /* CAKE_DTYPE_* of the reduced local output */
  int32_t transport_dtype; /* CAKE_DTYPE_* of partial sums crossing the link (world > 1) */
  int32_t strategy;     /* CAKE_RS_* (ignored when world == 1) */
  int32_t tile_m;       /* 128 */
  int32_t tile_n;       /* 64, 128 or 256 */
  int32_t rhs_layout;   /* 0 = rhs is [k_local, n] row-major (the reference layout),
                           1 = rhs is [n, k_local] row-major (pre-transposed) */
  int32_t wait_budget_ms; /* how long the slot reduction waits for a peer's data before it gives up
                             with CAKE_ERR_TIMEOUT; 0 = the default of 20 s */
} cake_matmul_rs_desc;

typedef struct cake_matmul_rs cake_matmul_rs;

int32_t cake_matmul_rs_create(const cake_matmul_rs_desc* desc, cake_matmul_rs** out);
int32_t cake_matmul_rs_destroy(cake_matmul_rs* plan);

/* Bytes of the partial buffer for CAKE_RS_LOCAL_PARTIAL (m * n * transport size). */
size_t cake_matmul_rs_partial_bytes(const cake_matmul_rs* plan);

/* CAKE_RS_P2P_OWNER_PUSH: bytes of this rank's receive slots (two parities x W sources x one local
 * output in the transport dtype, each padded to 128 bytes) and of its arrival flags (one 32-bit word
 * per source rank and quarter tile). */
size_t cake_matmul_rs_slot_bytes(const cake_matmul_rs* plan);
size_t cake_matmul_rs_flag_bytes(const cake_matmul_rs* plan);

/* CAKE_RS_P2P_OWNER_PUSH: the slot and flag buffers of every rank (entry [rank] is this rank's own
 * allocation -- slots 128-byte aligned, flags ZERO before the first enqueue, as cake_symm_alloc
 * returns them -- the others are IPC mappings). Called once before the first enqueue.
 *
 * Protocol. Call number e (1, 2, ...) writes its partial tiles into the slots of parity e & 1 and then
 * stores e into the owner's flag of each quarter tile (32 rows x tile_n columns) it has sent; the
 * reduction waits until all W flags of a quarter have reached e before it reads the quarter. Flags
 * only grow and a reduction consumes nothing, so a rank may run one call ahead of a slower peer, and
 * a reduction that ran out of its wait budget (CAKE_ERR_TIMEOUT from cake_matmul_rs_status, code 2,
 * detail1 = the source rank that was missing) can be enqueued again with
 * cake_matmul_rs_enqueue_reduce once the peer has caught up. Every rank must make the same sequence
 * of calls. */
int32_t cake_matmul_rs_bind_peers(cake_matmul_rs* plan, void* const* slots, void* const* flags);

/* lhs: bf16 [m, k_local]; rhs: bf16 per rhs_layout; out: world == 1 or P2P: the reduced local
 * output [m/W, n] or [m, n/W] in out_dtype; LOCAL_PARTIAL with world > 1: the owner-major partial
 * [W][out_rows][out_cols] in transport_dtype. */
int32_t cake_matmul_rs_enqueue(cake_matmul_rs* plan, const void* lhs, const void* rhs, void* out,
                               void* stream);

/* CAKE_RS_P2P_OWNER_PUSH only: the two halves of cake_matmul_rs_enqueue as separate kernels (the
 * contraction without its reduction warps, and cake_reduce_slots_sm100), so a host that drives
 * several mesh positions in one process (a test that emulates W ranks on one GPU, a single-process
 * multi-GPU driver) can enqueue every position's push before any reduction and never has one launch
 * wait on a later one. */
int32_t cake_matmul_rs_enqueue_push(cake_matmul_rs* plan, const void* lhs, const void* rhs,
                                    void* stream);
int32_t cake_matmul_rs_enqueue_reduce(cake_matmul_rs* plan, void* out, void* stream);

/* Same computation with HOST buffers: copies lhs and rhs to device staging buffers owned by the
 * plan, enqueues, copies the local output back and synchronises the stream. world == 1 or P2P.
 * At world == 1, when lhs is large enough (blocks of whole tiles and at least 8 MiB each), the
 * matrix goes through in up to 8 blocks of rows on two copy streams of the plan's own, so that a
 * block is contracted while the next one arrives and the previous one leaves; the output bits are
 * those of one enqueue. Pinned host buffers are needed for that overlap, not for correctness. */
int32_t cake_matmul_rs_run_host(cake_matmul_rs* plan, const void* lhs_host, const void* rhs_host,
                                void* out_host, void* stream);

/* Reads (and clears) the device status word; synchronises the stream first. */
int32_t cake_matmul_rs_status(cake_matmul_rs* plan, void* stream, cake_status* out);

/* Number of kernels the last enqueue launched (for launch accounting). */
int32_t cake_matmul_rs_launches_per_enqueue(const cake_matmul_rs* plan);

/* ---------------------------------------------------------------- ragged paged attention
 * Replaces FusedRpaPlan.invoke / OwnedRpaDecodeCorePlan.build
 * (src/tpu_cake/rpa_lowering.py:232-273,900-963), whose device code is _owned_rpa_kernel_loop
 * (src/tpu_cake/rpa_owned_kernel.py:85-960), and gives the prototype op
 * tpu_schedule.ragged_paged_attention (src/tpu_cake/dialects/tpu_schedule.py:2003-2103) a lowering.
 */

#define CAKE_RPA_CACHE_SEPARATE 0 /* key_cache, value_cache: [pages, page_size, kv_heads, head_dim] */
#define CAKE_RPA_CACHE_FUSED 1    /* [pages, page_size, 2*kv_heads/2, 2, head_dim_padded]; head h's K at
                                     interleaved index 2h, V at 2h+1 */
#define CAKE_RPA_TABLE_2D 0       /* page_table[num_seqs, max_pages], token t -> page_table[s, t/ps] */
#define CAKE_RPA_TABLE_FLAT 1     /* page_indices flat; sequence s starts at cu_kv_lens[s] / ps */

typedef struct cake_rpa_desc {
  int32_t num_seqs;
  int32_t num_q_tokens;   /* sum of query lengths (== num_seqs for pure decode; larger: cake_rpa_mixed_enqueue) */
  int32_t q_heads;
  int32_t kv_heads;
  int32_t head_dim;       /* 128 */
  int32_t head_dim_padded;/* fused cache only; == head_dim for the separate layout */
  int32_t page_size;      /* tokens per page: 1, 2, 4, 8, 16 or 32 */
  int32_t cache_layout;   /* CAKE_RPA_CACHE_* */
  int32_t table_layout;   /* CAKE_RPA_TABLE_* */
  int32_t max_pages_per_seq; /* row pitch of the 2-D page table */
  int64_t total_pages;
  float sm_scale;
  int32_t bias_mode;      /* 0 = none, 1 = dense f32 bias[q_heads, bias_extent] indexed by key
                             position (prototype op), 2 = relative bias: states[tokens, q_heads, R]
                             (bf16) x projection[R, extent] (bf16) at distance kv_len-1-pos */
  int32_t bias_extent;
  int32_t rel_dim;        /* R for bias_mode 2 */
  int32_t update_cache;   /* 1 = first write new_k/new_v of each sequence at position kv_len-1 */
  int32_t kv_chunk_tokens;/* split-KV chunk; 0 = library default */
  int32_t wait_budget_ms; /* cake_rpa_decode_allgather_enqueue: how long the flag barrier waits for a
                             peer before it gives up with CAKE_ERR_TIMEOUT; 0 = the default of 20 s */
} cake_rpa_desc;

typedef struct cake_rpa cake_rpa;

int32_t cake_rpa_create(const cake_rpa_desc* desc, cake_rpa** out);
int32_t cake_rpa_destroy(cake_rpa* plan);

/* Scratch the decode needs for split-KV partial results (bytes, device memory). */
size_t cake_rpa_workspace_bytes(const cake_rpa* plan);

/* Pure decode (one query token per sequence).
 * q, out: bf16 [num_seqs, q_heads, head_dim] (out may alias q);
 * new_k, new_v: bf16 [num_seqs, kv_heads, head_dim] or NULL when update_cache == 0;
 * cache0: key cache (separate) or fused cache; cache1: value cache or NULL;
 * kv_lens: i32 [num_seqs]; page_table: i32 per table_layout; cu_kv_lens: i32 [num_seqs+1] (flat
 * layout) or NULL; bias0 / bias1 per bias_mode or NULL. */
int32_t cake_rpa_decode_enqueue(cake_rpa* plan, const void* q, const void* new_k, const void* new_v,
                                void* cache0, void* cache1, const int32_t* kv_lens,
                                const int32_t* page_table, const int32_t* cu_kv_lens,
                                const void* bias0, const void* bias1, void* out, void* workspace,
                                void* stream);

/* Ragged batch: sequences [0, num_decode_seqs) have one query token each and come first (the
 * reference's `distribution` order, src/tpu_cake/rpa_owned_kernel.py:58-67); the others are prefill
 * sequences whose q query tokens are the LAST q of their kv_len positions (causal: query token i
 * sees positions 0..kv_len-q+i). The reference lowers decode batches only
 * (src/tpu_cake/rpa_lowering.py:71-95 rejects anything else), so this call has the wrapped kernel's
 * semantics (causal=1, src/tpu_cake/rpa_lowering.py:232-273) but no reference test behind it.
 * q, out: bf16 [num_q_tokens, q_heads, 128]; new_k, new_v: bf16 [num_q_tokens, kv_heads, 128] (written
 * into the cache first when update_cache == 1); cu_q_lens: i32 [num_seqs+1] on the device;
 * num_decode_seqs: host value. Needs head_dim 128, bias_mode 0 and the fused cache layout. The decode sequences run through
 * the decode kernels, the others through the tcgen05 prefill kernel. */
int32_t cake_rpa_mixed_enqueue(cake_rpa* plan, const void* q, const void* new_k, const void* new_v,
                               void* cache0, void* cache1, const int32_t* kv_lens,
                               const int32_t* page_table, const int32_t* cu_kv_lens,
                               const int32_t* cu_q_lens, int32_t num_decode_seqs, void* out,
                               void* workspace, void* stream);

/* Decode of this rank's KV-head shard with the all-gather of the outputs fused in: every output
 * row is written straight into the gathered buffer of every rank over peer memory (P2P stores), then
 * a one-warp kernel publishes an epoch to every rank's flag array and, if `wait` is non-zero, waits
 * (bounded) until every rank has published. Replaces the "outputs stay sharded" end of the reference's
 * shard_map (src/tpu_cake/rpa_lowering.py:552-558) plus the all-gather the sharded configuration asks
 * for. gathered[r]: rank r's [2][world][num_seqs][q_heads][head_dim] bf16 buffer (q_heads = this
 * shard's query heads): the n-th call on a plan (n = 1, 2, ...) fills half n & 1 on every rank, so a
 * rank that runs one call ahead of a peer never overwrites what the peer's consumer of the previous
 * call -- ordered on the peer's stream after that call -- is still reading. Every rank must make the
 * same sequence of calls. flags[r]: rank r's CAKE_MAX_WORLD x uint64 array, zero before the first
 * call; entries [rank] are this rank's own allocations, the others peer mappings. `wait` = 0 lets a
 * host that drives several ranks from one process enqueue every rank before anybody waits. If a peer
 * never publishes, the wait gives up after wait_budget_ms (cake_rpa_status: CAKE_ERR_TIMEOUT, code 2,
 * detail1 = the missing rank). The first call allocates a 64-byte device table. */
int32_t cake_rpa_decode_allgather_enqueue(cake_rpa* plan, const void* q, const void* new_k,
                                          const void* new_v, void* cache0, void* cache1,
                                          const int32_t* kv_lens, const int32_t* page_table,
                                          const int32_t* cu_kv_lens, const void* bias0,
                                          const void* bias1, void* const* gathered,
                                          void* const* flags, int32_t world, int32_t rank,
                                          int32_t wait, void* workspace, void* stream);

/* Decode for hosts that may not allocate device memory. No counterpart in the reference: its
 * kernels get their scratch from the JAX runtime.
 *
 * Who needs it: a plugin inside a serving engine that owns the only device allocator and hands the
 * plugin fixed input and output buffers, or a serving loop whose memory pool is frozen after
 * start-up (an allocation there is refused, or stalls the whole device mid-request). Such a host
 * cannot provide the split-KV workspace cake_rpa_decode_enqueue asks for, and cannot call
 * cake_rpa_create either (it allocates a status word). This one call needs neither: it takes the
 * descriptor directly, keeps its scratch in an array built into the library
 * (CAKE_RPA_STATIC_SCRATCH_BYTES per GPU that loads the library, held until the process exits), and
 * calls no cudaMalloc, cudaFree or other allocating routine.
 *
 * Arguments are those of cake_rpa_decode_enqueue without the workspace. status_device is an
 * optional caller-owned device buffer of 4 int32 (zeroed by the caller) that receives the
 * cake_status fields if a device-side check fails; pass NULL to ignore.
 *
 * Limits and rules:
 *   - A shape whose scratch would exceed CAKE_RPA_STATIC_SCRATCH_BYTES is rejected with
 *     CAKE_ERR_UNSUPPORTED (the message states the bytes needed). The need grows with
 *     (page-table extent * page_size / kv_chunk_tokens + num_seqs) * q_heads * 520 bytes.
 *   - The first call on each device looks up the array's device address (one-time set-up); make
 *     that first call before any stream capture begins.
 *   - All calls on a device share the one array and it keeps the previous call's contents. Every
 *     call rewrites what it later reads, so calls that run one after another are independent, but
 *     two calls whose kernels overlap on the GPU (different streams) race on it: serialise them. */
#define CAKE_RPA_STATIC_SCRATCH_BYTES (16u << 20)
int32_t cake_rpa_decode_static_scratch(const cake_rpa_desc* desc, const void* q, const void* new_k,
                                       const void* new_v, void* cache0, void* cache1,
                                       const int32_t* kv_lens, const int32_t* page_table,
                                       const int32_t* cu_kv_lens, const void* bias0,
                                       const void* bias1, void* out, int32_t* status_device,
                                       void* stream);

int32_t cake_rpa_status(cake_rpa* plan, void* stream, cake_status* out);
int32_t cake_rpa_launches_per_enqueue(const cake_rpa* plan);

#ifdef __cplusplus
}
#endif
#endif /* CAKE_ABI_H_ */
