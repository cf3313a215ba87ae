/*
 * lrqk_sm100.h -- C ABI of liblrqk_sm100.so: the LRQK prefill-factorisation and
 * decode-time selection / attention path as CUDA kernels for NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Plain C: pointers, sizes, POD structs.  No C++ or torch types cross this line.
 *   - Every compute entry point enqueues work on the CUDA stream it is given and
 *     returns at once: 0 (LRQK_OK) or a negative LRQK_E* code (see lrqk_strerror).
 *     Nothing here synchronises the stream, and -- unless an entry says otherwise --
 *     nothing allocates: the caller owns every buffer, including scratch space whose
 *     size the matching *_workspace_bytes() function reports.
 *   - "device pointer" means an address a kernel on the current device can
 *     dereference.  The host K|V store is page-locked host memory; its
 *     device-visible address (lrqk_host_device_ptr) is what the structs carry.
 *   - All tensors are dense and row-major in the shapes written beside them.
 *     Shapes use: B batch, Hq query heads, Hkv key/value heads, G = Hq/Hkv,
 *     N = B*Hq, d head dim, r rank, k resident (selected) rows, m recent-token
 *     ("lite") rows.  Query head h reads KV head h / G.
 *   - There is no CPU fallback: on a machine without an sm_100 device every compute
 *     entry returns LRQK_ENODEVICE.
 *
 * Each entry cites the interface of the reference project (tenghuilee/LRQK, paths
 * relative to its checkout) that it stands in for.
 */
#ifndef LRQK_SM100_H_
#define LRQK_SM100_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *lrqk_stream_t; /* a cudaStream_t */

enum {
  LRQK_OK = 0,
  LRQK_EINVAL = -1,       /* null pointer, non-positive size, inconsistent shapes */
  LRQK_ECAPACITY = -2,    /* an index or length exceeds the capacity given        */
  LRQK_EUNSUPPORTED = -3, /* shape or dtype outside what the kernels are built for */
  LRQK_ELAUNCH = -4,      /* the CUDA runtime refused a launch or an API call     */
  LRQK_ETIMEOUT = -5,     /* a bounded device-side wait ran out                   */
  LRQK_ENODEVICE = -6,    /* no sm_100 device is current                          */
  LRQK_ENOMEM = -7        /* host allocation failed                               */
};

enum { LRQK_F32 = 0, LRQK_BF16 = 1 };

const char *lrqk_version(void);
const char *lrqk_strerror(int code);
/* 1 when the current CUDA device is compute capability 10.x, else 0. */
int lrqk_device_supported(void);
/* Text of the last CUDA runtime error seen by this library on the calling thread. */
const char *lrqk_last_cuda_error(void);

/* ------------------------------------------------------------------------------------
 * Page-locked, device-mapped host memory for the K|V store.
 * Stands in for torch.empty(..., pin_memory=True) of AutoIncreaseTensorSharedKV
 * (lrqk_attention.py:883-888, :1088-1094).  The memory is zero-filled, portable across devices and
 * addressable by kernels through lrqk_host_device_ptr.  (Anonymous huge-page memory registered with
 * the driver where that works -- about three times quicker to obtain than cudaHostAlloc -- else
 * cudaHostAlloc.)  These and lrqk_peer_buffer_create are the only entries that allocate.
 * ---------------------------------------------------------------------------------- */
int lrqk_host_alloc(void **host_ptr, size_t bytes);
int lrqk_host_free(void *host_ptr);
int lrqk_host_device_ptr(void *host_ptr, void **device_ptr);

/* ------------------------------------------------------------------------------------
 * State of one layer (one LightAttentionIndicesFactory, lrqk_attention.py:1052-1111).
 * All pointers are device pointers owned by the caller.
 * ---------------------------------------------------------------------------------- */
typedef struct lrqk_layer {
  int32_t dtype;          /* LRQK_F32 / LRQK_BF16: element type of every tensor below   */
  int32_t bsz, q_heads, kv_heads, head_dim;
  int32_t r, k, m;        /* rank, attn_topk, num_lite_tokens                            */
  int64_t a_capacity;     /* rows allocated per head in A_K (zero-initialised, :888)      */
  int64_t host_capacity;  /* rows allocated per (b, kv head) in the host store (:113)     */
  void *A_K;              /* [B,Hq,a_capacity,r]   rank-r key factors, all tokens         */
  void *B_Q;              /* [B,Hq,r,d]                                                   */
  void *B_K;              /* [B,Hq,r,d]                                                   */
  void *K_res;            /* [B,Hq,k+m,d]  resident keys: k selected slots, then m lite   */
  void *V_res;            /* [B,Hq,k+m,d]                                                 */
  int32_t *table;         /* [B,Hq,k]   token position held by each selected slot         */
  int32_t *lite_pos;      /* [m]        token position held by each lite slot             */
  void *host_kv;          /* device-visible address of host [B,Hkv,host_capacity,2d], K|V */
  float weights[4];       /* lambda_Q, lambda_K of the prompt factorisation, lambda_dec_q,
                             lambda_dec_k of the decode step (:1040, :1066-1072); each >= 0.
                             The reference's cache leaves all four at 1.                   */
} lrqk_layer;

/* One missed row: resident slot `slot` of head `head` (= b*Hq + h) must be refilled with
 * token position `pos` from the host store. */
typedef struct lrqk_miss {
  int32_t head, slot, pos;
} lrqk_miss;

/* ------------------------------------------------------------------------------------
 * Lite-ring write (+ optional flush of the ring to the host store).
 * Replaces LightAttentionIndicesFactory._append / __set_lite (lrqk_attention.py:1133-1135,
 * :1174-1196) and AutoIncreaseTensorSharedKV.append of the ring (:959-963, :1124-1131).
 *   k_new, v_new : [B,Hkv,d]   the step's key / value
 *   lite_slot    : ring slot written (K_res/V_res row k + lite_slot of all G heads of a group)
 *   position     : token position stored into lite_pos[lite_slot]
 *   flush_rows   : 0, or m when this write filled the ring: the ring of every KV head is then
 *                  copied, in slot order, to host rows [host_row, host_row + m) as K|V
 * ---------------------------------------------------------------------------------- */
int lrqk_lite_append(const lrqk_layer *L, const void *k_new, const void *v_new, int32_t lite_slot,
                     int32_t position, int32_t flush_rows, int64_t host_row, lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Rank-r projection of the step's q, k and update of B_Q, B_K.
 * Replaces _get_A_K_hitted_with_lite (lrqk_attention.py:1156-1171), cast_lrqk_decode /
 * _lrqk_decode_inv_w1 / _lrqk_decode_gd_B_lr (:522-628, :651-665, :803-839) and the
 * sync_cache append of k_hat (:1208-1233); with L->weights[2] or [3] (lambda_dec_q, lambda_dec_k)
 * different from 1, the weighted form _lrqk_decode_inv (:433-519) -- the same kernel, the active
 * set's sums scaled by lambda_dec_k, the new token's own q k^T term by lambda_dec_q.
 *   q        : [B,Hq,d], k_new: [B,Hkv,d]
 *   append_row : row of A_K that receives k_hat (the new token's position)
 *   q_hat    : out [B,Hq,r] in L->dtype
 *   iters_out: optional device int32[1], number of alternations actually applied
 * The active set is the k table entries followed by the m lite positions; A_K rows are
 * read from the capacity buffer, so the row of the token being appended reads as zero.
 * The early exit "mse(k_hat, k_hat') < tol" is a mean over ALL heads, as in the
 * reference (:603-609); it is evaluated on the device, without a host round trip.
 * Status: the bounded waits of the kernel (bulk copies of the resident keys, tensor-core completion)
 * record LRQK_ETIMEOUT in the int32 word lrqk_decode_project_update_status_word() points at (the last
 * 16 bytes of the workspace); zero-fill the workspace before its first use.
 * ---------------------------------------------------------------------------------- */
size_t lrqk_decode_project_update_workspace_bytes(const lrqk_layer *L, int32_t max_iter);
/* The two halves of lrqk_decode_project_update as separate calls, for callers that want to place (or time) them
 * separately -- lrqk_layer_step runs the first as its own kernel and the second inside the scoring kernel.
 * lrqk_decode_project: the alternating solves (:555-609); leaves every alternation's (q_hat, k_hat, squared
 * change) in `workspace` and touches nothing else.  lrqk_decode_update: the early-exit decision over all heads
 * (:603-609) from those, then B_Q, B_K (:612-626), q_hat and the new row of A_K.  Same workspace, same max_iter. */
int lrqk_decode_project(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter,
                        int64_t append_row, void *q_hat, void *workspace, lrqk_stream_t stream);
int lrqk_decode_update(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter, float tol,
                       int64_t append_row, void *q_hat, int32_t *iters_out, void *workspace,
                       lrqk_stream_t stream);
int32_t *lrqk_decode_project_update_status_word(const lrqk_layer *L, int32_t max_iter, void *workspace);
int lrqk_decode_project_update(const lrqk_layer *L, const void *q, const void *k_new, int32_t max_iter,
                               float tol, int64_t append_row, void *q_hat, int32_t *iters_out,
                               void *workspace, lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Proxy scores over the first `candidates` rows of A_K and top-k, fused.
 * Replaces compute_hit_indices (lrqk_attention.py:1235-1273: matmul, torch.topk, torch.sort).
 *   q_hat      : [B,Hq,r] in L->dtype
 *   candidates : c, k < c <= a_capacity
 *   wanted     : out [B,Hq,k] int32, ascending.  Scores are fp32 dot products of the stored
 *                operands; of equal scores the lower position wins (-0 equals +0).
 *   scores_out : optional [B,Hq,scores_stride] fp32 copy of the scores (testing)
 *   workspace  : optional scratch of lrqk_score_topk_workspace_bytes(L, largest candidate count to come).
 *                With few heads (a rank's share of a head-sharded layer) the scoring is cut into two
 *                kernels -- keys formed on all SMs into this scratch, then the selection -- which is quicker
 *                than clusters that cover a fraction of the GPU; that function returns 0 where the one-kernel
 *                plan is the better one.  NULL: always one kernel.  The selection is the same either way.
 * ---------------------------------------------------------------------------------- */
size_t lrqk_score_topk_workspace_bytes(const lrqk_layer *L, int64_t max_candidates);
int lrqk_score_topk(const lrqk_layer *L, const void *q_hat, int64_t candidates, int32_t *wanted,
                    float *scores_out, int64_t scores_stride, void *workspace, size_t workspace_bytes,
                    lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Hit/miss difference of `wanted` against the slot table, in place.
 * Replaces only_indices_in_cpu (lrqk_attention.py:1275-1315) and the index builder
 * _take_along_dim_with_mask_python_indices (:71-98).
 *   wanted     : [B,Hq,k] ascending, duplicate-free
 *   mask       : out [B,Hq,k] uint8, 1 = slot refilled
 *   miss_count : out [B,Hq] int32
 *   list       : out, room for B*Hq*k entries; *list_len (device int32, must be 0 on entry)
 *                receives the number of entries.  Entry order across heads is unspecified.
 *   status     : device int32[1]; set non-zero if a head's evicted and missing counts differ
 * ---------------------------------------------------------------------------------- */
int lrqk_slot_diff(const lrqk_layer *L, const int32_t *wanted, uint8_t *mask, int32_t *miss_count,
                   lrqk_miss *list, int32_t *list_len, int32_t *status, lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Fetch of the missed rows from the host store straight into their slots.
 * Replaces take_along_dim_with_mask_python -> cpp_kernel.d0_index_select -> .to(cuda)
 * (lrqk_attention.py:101-117, cpp_kernel/__init__.py:7-16,
 * cpp_kernel/take_along_dim_grouped.cpp:133-183) and the masked scatter (:1603-1608).
 * Reads *list_len on the device; no host synchronisation.
 * ---------------------------------------------------------------------------------- */
int lrqk_miss_gather(const lrqk_layer *L, const lrqk_miss *list, const int32_t *list_len,
                     lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Exact attention of one query per head over the first `rows` resident rows.
 * Replaces flash_attn_with_kvcache(q, k, v, causal=True) with one query
 * (lrqk_attention.py:2326-2327; Qwen2/Mistral :2205-2216, :2438-2449).
 *   q   : [B,Hq,d];  out : [B,Hq,d] in L->dtype;  scale: 1/sqrt(d) in the reference
 *   workspace must be zero-filled before its first use; the kernel leaves it reusable.
 *   Status: the kernel's one bounded wait (for the bulk copy of its keys) records LRQK_ETIMEOUT in the int32
 *   word that lrqk_flash_decode_status_word() points at (inside the workspace); it stays set until the
 *   caller clears it.  lrqk_layer_step uses the same word.
 * ---------------------------------------------------------------------------------- */
size_t lrqk_flash_decode_workspace_bytes(const lrqk_layer *L, int32_t rows);
int32_t *lrqk_flash_decode_status_word(const lrqk_layer *L, void *workspace);
int lrqk_flash_decode(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale,
                      void *workspace, lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * The same attention for callers that can neither allocate nor pass a workspace.
 * No counterpart in the reference: it exists for hosts whose device memory is entirely owned by
 * their own pool at call time (a serving runtime's plugin hook, a loop whose rules forbid
 * allocator calls) and that therefore cannot satisfy lrqk_flash_decode's workspace argument.
 * The scratch is an array compiled into the library (lrqk_flash_decode_static_capacity_bytes(),
 * 4 MiB, resident on every GPU that loads the library until the process exits).  This entry and
 * everything it calls allocate nothing.
 *   - Limit: B*Hq heads times the split count chosen for `rows` (one split per 32 KiB of keys)
 *     times 520 bytes must fit the array: 470 heads at 2112 bf16 rows of head_dim 128, 240 heads at
 *     4224 rows; larger shapes return LRQK_ECAPACITY and lrqk_last_cuda_error() says how many
 *     bytes were needed.
 *   - The first call on a device looks up the array's device address (once per device, with that
 *     device current); make that first call outside any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents; the entry clears
 *     the part that must start at zero on `stream` before launching.  Two calls that can overlap
 *     on the GPU (different streams, no ordering between them) race on it: serialise them.
 *   - Status: like lrqk_flash_decode, a bounded wait that runs out leaves LRQK_ETIMEOUT in a word of the
 *     scratch; the next call clears it.  lrqk_flash_decode_static_status() copies the word of the last call
 *     on the current device to `status_out` (host memory, page-locked if the copy is to be asynchronous)
 *     on `stream`; read it after synchronising that stream.  It allocates nothing either.
 * ---------------------------------------------------------------------------------- */
size_t lrqk_flash_decode_static_capacity_bytes(void);
int lrqk_flash_decode_static_status(int32_t *status_out, lrqk_stream_t stream);
int lrqk_flash_decode_static(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale,
                             lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Exchange of attention outputs between the ranks that shard a layer's KV heads (one process
 * per GPU of one node).  The reference runs on a single GPU and has no counterpart; the entry
 * points below stand where its attention output tensor (lrqk_attention.py:2326-2334) is handed
 * to the output projection, which needs the rows of ALL heads.
 *
 * Every rank owns one exchange buffer, made visible to its peers by CUDA IPC:
 *     data  [2][world][heads_per_rank][d]  elements of the layer dtype   (two alternating halves)
 *     flags [2][world] int32, 256-byte aligned behind the data            (arrival words)
 * A push with sequence number seq (1, 2, 3, ...) uses half seq & 1.  The attention kernel of
 * rank r stores each finished output row into slot [seq & 1][r] of EVERY rank's buffer with plain
 * peer stores over NVLink and, once all its heads are done, release-stores seq into
 * flags[seq & 1][r] of every rank.  No multicast object and no collective library is involved.
 * A rank may run at most one push ahead of its slowest peer, which holds whenever every rank
 * waits for push seq (lrqk_allgather_wait) before it issues push seq + 1.
 * ---------------------------------------------------------------------------------- */
#define LRQK_MAX_PEERS 8
typedef struct lrqk_peer_group {
  int32_t world, rank;
  int32_t heads_per_rank;          /* B * Hq of one rank's shard (the same on all ranks)       */
  int32_t head_dim, dtype;
  void *base[LRQK_MAX_PEERS];      /* exchange buffer of every rank as seen from this device   */
  int32_t *local_counter;          /* device int32[1] of this rank, zero before the first push */
} lrqk_peer_group;

/* Bytes of one rank's exchange buffer (data and flags). */
size_t lrqk_peer_buffer_bytes(int32_t world, int32_t heads_per_rank, int32_t head_dim, int32_t dtype);
/* cudaMalloc + zero-fill of an exchange buffer and its 64-byte IPC handle (allocates; set-up only). */
int lrqk_peer_buffer_create(size_t bytes, void **dev_ptr, unsigned char handle[64]);
/* Map a peer's buffer from its handle / undo that / free one's own buffer. */
int lrqk_peer_buffer_open(const unsigned char handle[64], void **dev_ptr);
int lrqk_peer_buffer_close(void *dev_ptr);
int lrqk_peer_buffer_destroy(void *dev_ptr);

/* lrqk_flash_decode whose epilogue also pushes the output rows to every rank of `g`.
 * `out` may be NULL when only the exchange buffer is wanted. */
int lrqk_flash_decode_push(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale,
                           void *workspace, const lrqk_peer_group *g, int32_t seq, lrqk_stream_t stream);
/* Miss fetch and attention in ONE kernel: lrqk_miss_gather (driven by `mask`, the byte per slot that
 * lrqk_slot_diff or the step's scoring kernel wrote, and the slot table it updated) followed by
 * lrqk_flash_decode over all k + m rows (or lrqk_flash_decode_push when `g` is not NULL; `out` may
 * then be NULL) -- with the same results bit for bit: the thread that attends to a refilled slot
 * reads that row from the host store itself (take_along_dim_with_mask + index_put_ + the attention
 * call of the reference, lrqk_attention.py:1570-1613, in one pass), and stores it into K_res/V_res
 * on the side.  lrqk_layer_step uses it whenever the step ends in attention. */
int lrqk_fetch_attend(const lrqk_layer *L, const uint8_t *mask, const void *q, void *out, float scale,
                      void *workspace, const struct lrqk_peer_group *g, int32_t seq, lrqk_stream_t stream);
/* Wait (bounded) until push `seq` of every rank has arrived in this rank's buffer, then copy the
 * gathered rows [world][heads_per_rank][d] to gathered_out if it is not NULL.  If the wait runs
 * out, *status (device int32) is set to LRQK_ETIMEOUT and the copy is skipped; the kernel always
 * returns, so the stream and the context stay usable.  In that case gathered_out is filled with NaNs
 * (all-ones bit patterns) instead of being left as it was. */
int lrqk_allgather_wait(const lrqk_peer_group *g, int32_t seq, void *gathered_out, int32_t *status,
                        lrqk_stream_t stream);
/* How often lrqk_allgather_wait polls an arrival word (about 1 us per poll) before it gives up;
 * the default, 2^22, is a few seconds.  Process-wide; applies to waits enqueued afterwards. */
int lrqk_peer_set_wait_polls(uint32_t polls);

/* ------------------------------------------------------------------------------------
 * One whole decode step of a layer: the six calls above in the reference's order
 * (LightAttentionIndicesFactory.decode, lrqk_attention.py:1506-1613, followed by the
 * attention call).  Host-side counters (ring slot, positions, candidate count) are the
 * caller's, exactly as they are Python attributes in the reference.
 * ---------------------------------------------------------------------------------- */
struct lrqk_peer_group;
typedef struct lrqk_step_args {
  const void *q;          /* [B,Hq,d]  */
  const void *k_new;      /* [B,Hkv,d] */
  const void *v_new;      /* [B,Hkv,d] */
  void *attn_out;         /* [B,Hq,d], may be NULL to skip attention */
  int32_t lite_slot;      /* ring slot this step writes                          */
  int32_t position;       /* token position of the new token (= current length)  */
  int32_t flush_rows;     /* m when this step fills the ring, else 0             */
  int64_t host_row;       /* first host row of a flush                           */
  int64_t candidates;     /* c = oldest lite position - 1 after the ring write   */
  int32_t max_iter;       /* decode alternations                                 */
  float tol;
  float scale;            /* softmax scale                                       */
  void *q_hat;            /* out [B,Hq,r]                                        */
  int32_t *wanted;        /* out [B,Hq,k]                                        */
  uint8_t *mask;          /* out [B,Hq,k]                                        */
  int32_t *miss_count;    /* out [B,Hq]                                          */
  lrqk_miss *miss_list;   /* scratch, B*Hq*k entries                             */
  int32_t *counters;      /* device int32[4]: [0] list length, [1] status, [2] iterations, [3] spare */
  void *project_workspace;
  void *attn_workspace;
  const struct lrqk_peer_group *peers; /* NULL, or the ranks that receive this layer's attention output */
  int32_t push_seq;       /* sequence number of this push (see lrqk_flash_decode_push)  */
  void *score_workspace;  /* NULL, or scratch of lrqk_score_topk_workspace_bytes() for the scoring stage */
  size_t score_workspace_bytes;
  void *gathered_out;     /* with peers: where lrqk_allgather_wait puts all ranks' rows (may be NULL)          */
  int32_t *wait_status;   /* with peers: non-NULL makes the step end with lrqk_allgather_wait(peers, push_seq,
                             gathered_out, wait_status), so a head-sharded layer-step is ONE call              */
} lrqk_step_args;

int lrqk_layer_step(const lrqk_layer *L, const lrqk_step_args *a, lrqk_stream_t stream);
/* Number of kernels that call enqueues for these arguments (3 to 7: projection, [update], [key pass], scoring +
 * difference, miss fetch -- inside the attention kernel when the step ends in attention --, [ring flush],
 * [exchange wait]); negative LRQK_E* on bad arguments. */
int lrqk_layer_step_launches(const lrqk_layer *L, const lrqk_step_args *a);

/* ------------------------------------------------------------------------------------
 * The reference's native gather interface (pybind11 module take_along_dim_grouped,
 * cpp_kernel/take_along_dim_grouped.cpp:185-208), as device kernels that read the
 * page-locked host source directly.
 * ---------------------------------------------------------------------------------- */
/* dst[i,:] = src[rows[i],:]  -- d0_indices_select (:133-183).  dst, rows: device; src: device-
 * visible (host-mapped or device) memory; row_bytes a multiple of 16. */
int lrqk_d0_indices_select(void *dst, const void *src, const int64_t *rows, int64_t n_rows,
                           int64_t row_bytes, int64_t src_rows, lrqk_stream_t stream);
/* take_along_dim_with_mask (:13-124): src [B,Hkv,S,row_bytes], indices int64 and mask uint8
 * [B,Hkv,G,k]; dst receives the masked rows in row-major mask order; *n_out (device int64)
 * their number.  workspace: lrqk_take_along_dim_with_mask_workspace_bytes(). */
size_t lrqk_take_along_dim_with_mask_workspace_bytes(int64_t bsz, int64_t kv_heads, int64_t groups,
                                                     int64_t k);
int lrqk_take_along_dim_with_mask(void *dst, const void *src, const int64_t *indices,
                                  const uint8_t *mask, int64_t bsz, int64_t kv_heads, int64_t seq_len,
                                  int64_t groups, int64_t k, int64_t row_bytes, int64_t *n_out,
                                  void *workspace, lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * The patched attention forward's decode-time preamble (lrqk_attention.py:2254-2275: q_proj,
 * k_proj, v_proj -> view/transpose -> apply_rotary_pos_emb), after ONE fused projection: from
 * qkv [bsz, (q_heads + 2 kv_heads) * head_dim] (one new token per sequence; q heads, then k
 * heads, then v heads) and the position's cos, sin [cos_rows, head_dim] (cos_rows = bsz, or 1 when
 * all sequences are at the same position), writes the rotated q
 * [b_count, kvh_count * G, head_dim], rotated k and plain v [b_count, kvh_count, head_dim] of
 * batch entries b0 .. b0+b_count-1 and KV heads kvh0 .. kvh0+kvh_count-1 (a rank's shard; the
 * whole tensor with 0, bsz, 0, kv_heads).  Rotate-half form, x*cos + rotate_half(x)*sin, rounded
 * to `dtype` after each product and after the sum like the eager tensor operations.
 * ---------------------------------------------------------------------------------- */
int lrqk_rope_qkv(const void *qkv, const void *cos, const void *sin, int32_t cos_rows, int32_t dtype,
                  int32_t bsz, int32_t q_heads, int32_t kv_heads, int32_t head_dim, int32_t b0, int32_t b_count,
                  int32_t kvh0, int32_t kvh_count, void *q_out, void *k_out, void *v_out,
                  lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Element-wise glue of a decoder layer around the attention call, for the decode step (one token per
 * sequence), where every eager framework op is one launch of pure latency.  The reference leaves these to
 * the transformers modules (LlamaRMSNorm / Qwen2RMSNorm / MistralRMSNorm forward, the residual adds of the
 * decoder layer, `act_fn(gate_proj(x)) * up_proj(x)` of the MLP); these entries give the same rows with one
 * launch each, rounding where those tensor ops round.
 *   lrqk_add_rmsnorm: s = x + delta (delta may be NULL: s = x), rounded to `dtype`; optional sum_out = s;
 *                     normed_out = weight * dtype(s * rsqrt(mean(s^2) + eps));  x, delta, outs [rows, hidden]
 *   lrqk_swiglu     : out[r, i] = dtype(dtype(silu(gate_up[r, i])) * gate_up[r, inter + i]),
 *                     gate_up [rows, 2 * inter] (the fused gate|up projection), out [rows, inter]
 * ---------------------------------------------------------------------------------- */
int lrqk_add_rmsnorm(const void *x, const void *delta, const void *weight, float eps, int32_t dtype,
                     int32_t rows, int32_t hidden, void *sum_out, void *normed_out, lrqk_stream_t stream);
int lrqk_swiglu(const void *gate_up, int32_t dtype, int32_t rows, int32_t inter, void *out, lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Prompt-time helpers of LightAttentionIndicesFactory.prefill (lrqk_attention.py:1385-1504).
 * ---------------------------------------------------------------------------------- */
/* K|V rows of the prompt into the host store (KVcpu.append, :1469, :959-963):
 * keys, values [B,Hkv,S,d] -> host rows [host_row, host_row+S) of every (b, kv head). */
int lrqk_kv_pack_host(const lrqk_layer *L, const void *keys, const void *values, int64_t seq_len,
                      int64_t host_row, lrqk_stream_t stream);
/* Selected prompt rows into the resident slots, on the device (fetch_by_hit same-device
 * branch, :1339-1351) and the last m prompt tokens into the lite slots (:1493-1504):
 * K_res/V_res[n, s] = keys/values[b, kvh, table[n, s]] for s < k; slots k..k+m-1 receive
 * positions S-m..S-1, which are also written to lite_pos. */
int lrqk_prefill_fill_resident(const lrqk_layer *L, const void *keys, const void *values,
                               int64_t seq_len, lrqk_stream_t stream);

/* ------------------------------------------------------------------------------------
 * Prompt factorisation  Q ~ A_Q B_Q, K ~ A_K B_K with A_Q A_K^T ~ Q K^T.
 * Replaces cast_lrqk_prefill / _lrqk_prefill_inv_w1 (lrqk_attention.py:312-423, :772-800) and, when
 * L->weights[0] or [1] (lambda_Q, lambda_K) differs from 1, _lrqk_prefill_inv (:218-309), whose sweep
 * renews BOTH left factors from the factors it started with.
 *   Q [B,Hq,S,d], K [B,Hkv,S,d] in L->dtype (K is NOT expanded to the query heads)
 *   A_Q, A_K_init : fp32 [B,Hq,S,r] initial factors (see _init_AQ_AK, :187-209); overwritten
 *   sweeps, tol : max_iter[0], tol[0]; the stop test after a sweep is evaluated on the device
 * Outputs: L->A_K rows [0,S), L->B_Q, L->B_K in L->dtype; a_q_last [B,Hq,r] in L->dtype
 * (the last row of A_Q, the query of the prompt-time selection, :1471-1474);
 * sweeps_out optional device int32[1].
 * ---------------------------------------------------------------------------------- */
size_t lrqk_prefill_factorize_workspace_bytes(const lrqk_layer *L, int64_t seq_len);
int lrqk_prefill_factorize(const lrqk_layer *L, const void *Q, const void *K, float *A_Q,
                           float *A_K_init, int64_t seq_len, int32_t sweeps, float tol,
                           void *a_q_last, int32_t *sweeps_out, void *workspace,
                           lrqk_stream_t stream);

/* After lrqk_prefill_factorize (same L, seq_len, sweeps and workspace; sweeps_out as that call wrote it): copies
 * the d x r maps of the stopping sweep out of the workspace -- in fp32, A_Q = Q X_Q and A_K = K X_K -- to
 * x_q_out / x_k_out, fp32 [B,Hq,d,r]; either may be NULL.  For callers that want the full left factor of the
 * queries, which the reference's cast_lrqk_prefill returns (lrqk_attention.py:772-800) and the decode path never
 * needs beyond its last row. */
int lrqk_prefill_factor_maps(const lrqk_layer *L, int64_t seq_len, int32_t sweeps, const int32_t *sweeps_out,
                             const void *workspace, float *x_q_out, float *x_k_out, lrqk_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* LRQK_SM100_H_ */
