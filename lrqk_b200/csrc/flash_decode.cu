// Exact single-query attention over the resident rows, split over the row axis.
//
// Grid (splits, B*Hq), sized so that the whole grid is resident at once.  A CTA owns a contiguous
// run of rows of one head.  Everything it reads is requested before anything is waited for: one
// thread starts a bulk asynchronous copy (cp.async.bulk, completion on an mbarrier) that brings
// the run of K_res into shared memory, and every thread loads its share of V_res into registers.
// Scores are formed as soon as the keys have landed (a row spread over the lanes of a sub-warp,
// 16 bytes each), the softmax weights are taken against the run's maximum in base 2, and the
// weighted sum of the values follows from the registers.  One partial
// (unnormalised sum, maximum, weight sum) per split goes to the workspace; the CTA that finishes
// last for a head (an atomic ticket) folds the partials in split order, writes the output row and
// re-arms the ticket.  Runs longer than the staging buffers are processed in several rounds with
// the usual running-maximum rescale.
//
// The wait on the mbarrier is bounded: if it runs out, the CTA records it in the status word,
// contributes an empty partial and still takes its ticket, so nothing is left waiting.
//
// Miss fetch fused in (FETCH): a slot whose mask byte is set is refilled from the page-locked host
// store by the very thread that attends to it -- its 16-byte piece of the value row comes over the
// host link straight into the register the weighted sum reads, its piece of the key row by an
// asynchronous 16-byte copy into the staging buffer (this variant stages every key piece that way
// instead of one bulk copy), and both pieces are stored into the resident rows on the side.  Same threads, same pieces, same order
// of operations as the fetch kernel followed by this kernel without FETCH: bit-identical results,
// one launch and one pass over the missed rows fewer.
#include <math.h>
#include <stdio.h>

#include "common.cuh"
#include "peer.cuh"

namespace lrqk {
namespace {

constexpr int kAThreads = 256;
constexpr int kAWarps = kAThreads / 32;
constexpr int kMaxSplits = 64;
constexpr int kStageBytes = 32 * 1024;        // staging buffer for the keys of one round

struct AttnParams {
  const void *q, *K_res, *V_res;
  void *out;
  float *partial;     // [N][splits][D+2]
  int32_t *tickets;   // [N]
  int32_t *status;    // set to LRQK_ETIMEOUT if a bounded wait ran out
  int32_t slots;      // rows allocated per head (k + m)
  int32_t rows;       // rows attended
  int32_t splits, chunk;
  float scale_log2;   // softmax scale * log2(e)
  PushTargets push;   // world == 0: no exchange with other ranks
  // FETCH only: slots [0, k) with a set mask byte are refilled from host row table[slot]
  const uint8_t *mask;      // [N][k]
  const int32_t *table;     // [N][k]
  const char *host_kv;      // [B][Hkv][host_capacity][K row | V row]
  void *K_res_w, *V_res_w;
  int64_t host_capacity;
  int32_t k, q_heads, groups, kv_heads;
};

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}

template <typename T, int D, bool FETCH>
__global__ void __launch_bounds__(kAThreads, 4) flash_decode_kernel(AttnParams p) {
  constexpr int EPV = Elt<T>::kPerVec;            // elements per 16-byte vector
  constexpr int LPR = D / EPV;                    // lanes per row
  constexpr int GROUPS = kAThreads / LPR;         // rows handled side by side by the CTA
  constexpr int ROW_BYTES = D * (int)sizeof(T);
  constexpr int STAGE_ROWS = kStageBytes / ROW_BYTES;
  constexpr int RPT = STAGE_ROWS / GROUPS;        // rows per thread and round (8 for every supported shape)
  const int split = blockIdx.x, n = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lir = tid % LPR, grp = tid / LPR;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  T *sK = reinterpret_cast<T *>(smem_raw);                         // [STAGE_ROWS][D]; reused for the group sums
  float *s_w = reinterpret_cast<float *>(smem_raw + kStageBytes);  // [STAGE_ROWS] scores, then weights
  float *s_red = s_w + STAGE_ROWS;                                 // [kAWarps] block reduction
  uint64_t *bar = reinterpret_cast<uint64_t *>(s_red + kAWarps);
  __shared__ int is_last;

  const int r_begin = split * p.chunk;
  const int r_end = min(p.rows, r_begin + p.chunk);
  const char *Kg = reinterpret_cast<const char *>(p.K_res) + ((int64_t)n * p.slots) * ROW_BYTES;
  const char *Vg = reinterpret_cast<const char *>(p.V_res) + ((int64_t)n * p.slots) * ROW_BYTES + lir * 16;
  // FETCH: this head's mask and slot table, this thread's 16-byte piece of its KV head's host rows
  const uint8_t *mk = nullptr;
  const int32_t *tb = nullptr;
  const char *hrow = nullptr;
  char *Kw = nullptr, *Vw = nullptr;
  if constexpr (FETCH) {
    mk = p.mask + (int64_t)n * p.k;
    tb = p.table + (int64_t)n * p.k;
    const int b_idx = n / p.q_heads, h = n % p.q_heads;
    hrow = p.host_kv + ((int64_t)b_idx * p.kv_heads + h / p.groups) * p.host_capacity * (2 * ROW_BYTES) + lir * 16;
    Kw = reinterpret_cast<char *>(p.K_res_w) + ((int64_t)n * p.slots) * ROW_BYTES + lir * 16;
    Vw = reinterpret_cast<char *>(p.V_res_w) + ((int64_t)n * p.slots) * ROW_BYTES + lir * 16;
  }

  pdl_launch_dependents();
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();  // the rows this kernel reads are written by the kernels before it

  float m_run = -INFINITY, l_run = 0.0f;
  float2 acc[EPV / 2], qf[EPV / 2];  // pairs of neighbouring dimensions: two fused multiply-adds per instruction
#pragma unroll
  for (int e = 0; e < EPV / 2; ++e) acc[e] = make_float2(0.0f, 0.0f);
  bool timed_out = false;
  uint32_t parity = 0;

  for (int base = r_begin; base < r_end; base += STAGE_ROWS) {  // CTA-uniform trip count
    const int nrows = min(STAGE_ROWS, r_end - base);
    // everything this round reads is requested before anything is waited for: the keys by one bulk
    // copy into shared memory, the values straight into registers
    if constexpr (!FETCH) {
      if (tid == 0) {
        const uint32_t bytes = (uint32_t)nrows * ROW_BYTES;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(smem_addr(sK)), "l"(Kg + (int64_t)base * ROW_BYTES), "r"(bytes), "r"(smem_addr(bar)) : "memory");
      }
    }
    if (base == r_begin) {
      float raw[EPV];
      Elt<T>::unpack(ld16(reinterpret_cast<const T *>(p.q) + (int64_t)n * D + lir * EPV), raw);
#pragma unroll
      for (int e = 0; e < EPV / 2; ++e) qf[e] = make_float2(raw[2 * e] * p.scale_log2, raw[2 * e + 1] * p.scale_log2);
    }
    uint4 vv[RPT];
    uint32_t fetch_bits = 0;  // which of this thread's rows come from the host store
    if constexpr (FETCH) {
      // No bulk copy here: every thread brings its own 16-byte piece of each of its key rows into the
      // staging buffer with an asynchronous copy -- from the host store for a slot that is being refilled,
      // from the resident rows otherwise -- so that key and value of a missed row are requested together.
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int j = grp + i * GROUPS;
        const int slot = base + j;
        if (j < nrows) {
          int64_t pos = -1;
          if (slot < p.k) {  // mask byte and table entry are asked for together, not one after the other
            const uint8_t refill = mk[slot];
            const int32_t at = tb[slot];
            if (refill != 0) pos = at;
          }
          if (pos >= 0 && pos < p.host_capacity) {  // (a malformed entry is skipped, never dereferenced)
            const char *src = hrow + pos * (2 * ROW_BYTES);
            cp_async16(smem_addr(sK + (size_t)j * D + lir * EPV), src);
            vv[i] = ld16(src + ROW_BYTES);
            fetch_bits |= 1u << i;
          } else {
            cp_async16(smem_addr(sK + (size_t)j * D + lir * EPV), Kg + (int64_t)slot * ROW_BYTES + lir * 16);
            vv[i] = ld_stream16(Vg + (int64_t)slot * ROW_BYTES);
          }
        } else {
          vv[i] = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    } else {
#pragma unroll
      for (int i = 0; i < RPT; ++i) {
        const int j = grp + i * GROUPS;
        vv[i] = j < nrows ? ld_stream16(Vg + (int64_t)(base + j) * ROW_BYTES) : make_uint4(0u, 0u, 0u, 0u);
      }
      // ---- scores of this round -------------------------------------------------------------
      if (!mbar_wait_bounded(bar, parity)) timed_out = true;
    }
    float sc[RPT];
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int j = grp + i * GROUPS;
      float2 s2 = make_float2(0.0f, 0.0f);
      if (j < nrows) {
        float kf[EPV];
        Elt<T>::unpack(*reinterpret_cast<const uint4 *>(sK + (size_t)j * D + lir * EPV), kf);
#pragma unroll
        for (int e = 0; e < EPV / 2; ++e) s2 = __ffma2_rn(make_float2(kf[2 * e], kf[2 * e + 1]), qf[e], s2);
      }
      sc[i] = s2.x + s2.y;
    }
    // The RPT partial sums of a lane are folded over the LPR lanes of its row group by a
    // transposing butterfly: each step halves the number of values a lane carries, so the fold
    // costs RPT - 1 + log2(LPR / RPT) shuffles instead of RPT * log2(LPR).  Every lane of the
    // warp takes part in every shuffle.
    int mine = 0;  // which of the thread's rows this lane ends up holding the full score of
    {
      int o = LPR / 2;
#pragma unroll
      for (int half = RPT / 2; half >= 1; half >>= 1, o >>= 1) {
        const bool up = (lir & o) != 0;
#pragma unroll
        for (int i = 0; i < half; ++i) {
          const float send = up ? sc[i] : sc[i + half];
          const float keep = up ? sc[i + half] : sc[i];
          sc[i] = keep + __shfl_xor_sync(0xFFFFFFFFu, send, o);
        }
        if (up) mine += half;
      }
#pragma unroll
      for (; o >= 1; o >>= 1) sc[0] += __shfl_xor_sync(0xFFFFFFFFu, sc[0], o);
    }
    if constexpr (FETCH) {
      // ... and into the resident rows, for the steps to come
      if (fetch_bits) {
#pragma unroll
        for (int i = 0; i < RPT; ++i) {
          if (fetch_bits >> i & 1u) {
            const int j = grp + i * GROUPS;
            st16(Kw + (int64_t)(base + j) * ROW_BYTES, *reinterpret_cast<const uint4 *>(sK + (size_t)j * D + lir * EPV));
            st16(Vw + (int64_t)(base + j) * ROW_BYTES, vv[i]);
          }
        }
      }
    }
    float mx = -INFINITY;
    {
      const int j = grp + mine * GROUPS;
      if (j < nrows) {
        s_w[j] = sc[0];  // (lanes that hold the same row write the same value)
        mx = sc[0];
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    if (lane == 0) s_red[warp] = mx;
    __syncthreads();
#pragma unroll
    for (int w = 0; w < kAWarps; ++w) mx = fmaxf(mx, s_red[w]);
    const float m_new = fmaxf(m_run, mx);
    const float corr = exp2f(m_run - m_new);  // exp2f(-inf) = 0 in the first round
    // ---- weighted sum of the values -------------------------------------------------------
    l_run *= corr;
#pragma unroll
    for (int e = 0; e < EPV / 2; ++e) { acc[e].x *= corr; acc[e].y *= corr; }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int j = grp + i * GROUPS;
      if (j < nrows) {
        float vf[EPV];
        Elt<T>::unpack(vv[i], vf);
        const float w = exp2f(s_w[j] - m_new);
        l_run += w;
        const float2 w2 = make_float2(w, w);
#pragma unroll
        for (int e = 0; e < EPV / 2; ++e) acc[e] = __ffma2_rn(w2, make_float2(vf[2 * e], vf[2 * e + 1]), acc[e]);
      }
    }
    m_run = m_new;
    parity ^= 1u;
    __syncthreads();  // the key buffer, s_w and s_red are rewritten by the next round
  }
  if (timed_out) {  // contribute nothing rather than garbage
    atomicExch(p.status, (int32_t)LRQK_ETIMEOUT);
    m_run = -INFINITY; l_run = 0.0f;
#pragma unroll
    for (int e = 0; e < EPV / 2; ++e) acc[e] = make_float2(0.0f, 0.0f);
  }
  // fold the row groups in group order; the key buffer is free now
  float *g_acc = reinterpret_cast<float *>(sK);  // [GROUPS][D + 1]
#pragma unroll
  for (int e = 0; e < EPV / 2; ++e) {
    g_acc[grp * (D + 1) + lir * EPV + 2 * e] = acc[e].x;
    g_acc[grp * (D + 1) + lir * EPV + 2 * e + 1] = acc[e].y;
  }
  if (lir == 0) g_acc[grp * (D + 1) + D] = l_run;
  __syncthreads();
  float *part = p.partial + ((int64_t)n * p.splits + split) * (D + 2);
  for (int c = tid; c <= D; c += kAThreads) {
    float s = 0.0f;
#pragma unroll 8
    for (int g = 0; g < GROUPS; ++g) s += g_acc[g * (D + 1) + c];
    if (c < D) part[c] = s;
    else { part[D] = m_run; part[D + 1] = s; }
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    const int ticket = atomicAdd(&p.tickets[n], 1);
    is_last = ticket == p.splits - 1;
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // fold the partials of this head in split order.  They are first brought into shared memory by
  // all threads at once (one trip to memory), up to kFoldSplits splits at a time.
  constexpr int kFoldSplits = 32;
  float *buf = reinterpret_cast<float *>(smem_raw);  // [kFoldSplits][D + 2]
  const float *ph = p.partial + (int64_t)n * p.splits * (D + 2);
  float mx = -INFINITY, num = 0.0f, den = 0.0f;
  for (int s0 = 0; s0 < p.splits; s0 += kFoldSplits) {
    const int ns = min(kFoldSplits, p.splits - s0);
    __syncthreads();
    for (int i = tid; i < ns * (D + 2); i += kAThreads) buf[i] = __ldcg(ph + (int64_t)s0 * (D + 2) + i);
    __syncthreads();
    if (tid < D) {
      for (int s = 0; s < ns; ++s) {
        const float ms = buf[s * (D + 2) + D];
        if (ms == -INFINITY) continue;
        const float mn = fmaxf(mx, ms);
        const float c0 = exp2f(mx - mn), c1 = exp2f(ms - mn);
        num = num * c0 + buf[s * (D + 2) + tid] * c1;
        den = den * c0 + buf[s * (D + 2) + D + 1] * c1;
        mx = mn;
      }
    }
  }
  if (tid < D) {
    const T val = Elt<T>::from_float(num / den);
    if (p.out) reinterpret_cast<T *>(p.out)[(int64_t)n * D + tid] = val;
    // exchange with the other ranks: the row goes into this rank's slot of every rank's buffer
    for (int r = 0; r < p.push.world; ++r) reinterpret_cast<T *>(p.push.data[r])[(int64_t)n * D + tid] = val;
  }
  if (p.push.world > 0) {
    __threadfence_system();  // the rows are out before this head is counted
    __syncthreads();
    if (tid == 0) {
      const int done = atomicAdd(p.push.local_counter, 1);
      if (done == p.push.heads - 1) {  // every head of this rank has been pushed: raise the arrival words
        *p.push.local_counter = 0;
        __threadfence_system();
        for (int r = 0; r < p.push.world; ++r)
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.push.flag[r]), "r"(p.push.seq) : "memory");
      }
    }
  }
  if (tid == 0) p.tickets[n] = 0;  // re-arm for the next call
}

// Rows per staging round for a row of `row_bytes`, and the split count for `rows` rows:
// one round per CTA while the split count allows it.
int plan_splits(int row_bytes, int rows) {
  const int stage_rows = kStageBytes / row_bytes;
  int splits = (rows + stage_rows - 1) / stage_rows;
  if (splits > kMaxSplits) splits = kMaxSplits;
  if (splits < 1) splits = 1;
  return splits;
}

constexpr size_t kAttnSmem = (size_t)kStageBytes + (kStageBytes / 128) * sizeof(float) + kAWarps * sizeof(float) + 16 + 128;

// Workspace layout: [n_heads] tickets, one status word, padding to 256 bytes, then the partials.
size_t ticket_region_bytes(int n_heads) { return ((size_t)(n_heads + 1) * sizeof(int32_t) + 255) / 256 * 256; }

int launch_flash_decode(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale, void *scratch,
                        cudaStream_t s, const lrqk_peer_group *g = nullptr, int32_t seq = 0,
                        const uint8_t *fetch_mask = nullptr) {
  const int n_heads = L->bsz * L->q_heads;
  AttnParams p;
  p.push.world = 0;
  p.mask = fetch_mask; p.table = L->table; p.host_kv = reinterpret_cast<const char *>(L->host_kv);
  p.K_res_w = L->K_res; p.V_res_w = L->V_res;
  p.host_capacity = L->host_capacity;
  p.k = L->k; p.q_heads = L->q_heads; p.kv_heads = L->kv_heads; p.groups = L->q_heads / L->kv_heads;
  if (g) {
    const size_t esz = elt_size(L->dtype);
    const size_t half = peer_data_bytes(g->world, g->heads_per_rank, g->head_dim, g->dtype) / 2;
    const size_t slot = (size_t)g->heads_per_rank * g->head_dim * esz;
    for (int r = 0; r < g->world; ++r) {
      char *b = reinterpret_cast<char *>(g->base[r]);
      p.push.data[r] = b + (size_t)(seq & 1) * half + (size_t)g->rank * slot;
      p.push.flag[r] = reinterpret_cast<int32_t *>(b + 2 * half) + (seq & 1) * g->world + g->rank;
    }
    p.push.local_counter = g->local_counter;
    p.push.world = g->world;
    p.push.heads = n_heads;
    p.push.seq = seq;
  }
  p.q = q; p.K_res = L->K_res; p.V_res = L->V_res; p.out = out;
  p.tickets = reinterpret_cast<int32_t *>(scratch);
  p.status = p.tickets + n_heads;
  p.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(scratch) + ticket_region_bytes(n_heads));
  p.slots = L->k + L->m;
  p.rows = rows;
  p.splits = plan_splits((int)(L->head_dim * elt_size(L->dtype)), rows);
  p.chunk = (rows + p.splits - 1) / p.splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(p.splits, n_heads, 1);
#define LRQK_ATTN_LAUNCH(T, D)                                                                              \
  do {                                                                                                      \
    if (fetch_mask) {                                                                                       \
      auto kern = flash_decode_kernel<T, D, true>;                                                          \
      static SmemOptIn opt_in;                                                                              \
      LRQK_CUDA_TRY(opt_in.ensure(kern, kAttnSmem));                                                        \
      LRQK_CUDA_TRY(launch_dependent(kern, grid, dim3(kAThreads), kAttnSmem, s, 0, p));                     \
    } else {                                                                                                \
      auto kern = flash_decode_kernel<T, D, false>;                                                         \
      static SmemOptIn opt_in;                                                                              \
      LRQK_CUDA_TRY(opt_in.ensure(kern, kAttnSmem));                                                        \
      LRQK_CUDA_TRY(launch_dependent(kern, grid, dim3(kAThreads), kAttnSmem, s, 0, p));                     \
    }                                                                                                       \
  } while (0)
  if (L->head_dim == 128) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, LRQK_ATTN_LAUNCH(T, 128));
  } else if (L->head_dim == 64) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, LRQK_ATTN_LAUNCH(T, 64));
  } else {
    return LRQK_EUNSUPPORTED;
  }
#undef LRQK_ATTN_LAUNCH
  return LRQK_OK;
}

int check_attn_args(const lrqk_layer *L, const void *q, const void *out, int32_t rows) {
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!q || !L->K_res || !L->V_res) return LRQK_EINVAL;
  if (rows <= 0) return LRQK_EINVAL;
  if (rows > L->k + L->m) return LRQK_ECAPACITY;
  if (L->bsz * L->q_heads > 65535) return LRQK_EUNSUPPORTED;
  if (L->head_dim != 128 && L->head_dim != 64) return LRQK_EUNSUPPORTED;
  return LRQK_OK;
}

}  // namespace
}  // namespace lrqk

extern "C" size_t lrqk_flash_decode_workspace_bytes(const lrqk_layer *L, int32_t rows) {
  (void)rows;
  if (!L) return 0;
  const int n = L->bsz * L->q_heads;
  return lrqk::ticket_region_bytes(n) + (size_t)n * lrqk::kMaxSplits * (size_t)(L->head_dim + 2) * sizeof(float);
}

extern "C" int lrqk_flash_decode(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale,
                                 void *workspace, lrqk_stream_t stream) {
  using namespace lrqk;
  const int rc = check_attn_args(L, q, out, rows);
  if (rc != LRQK_OK) return rc;
  if (!workspace || !out) return LRQK_EINVAL;
  return launch_flash_decode(L, q, out, rows, scale, workspace, as_stream(stream));
}

extern "C" int lrqk_flash_decode_push(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale,
                                      void *workspace, const lrqk_peer_group *g, int32_t seq, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_attn_args(L, q, out, rows);
  if (rc != LRQK_OK) return rc;
  if (!workspace || seq < 1) return LRQK_EINVAL;
  rc = check_peer_group(g);
  if (rc != LRQK_OK) return rc;
  if (g->heads_per_rank != L->bsz * L->q_heads || g->head_dim != L->head_dim || g->dtype != L->dtype) return LRQK_EINVAL;
  return launch_flash_decode(L, q, out, rows, scale, workspace, as_stream(stream), g, seq);
}

extern "C" int lrqk_fetch_attend(const lrqk_layer *L, const uint8_t *mask, const void *q, void *out, float scale,
                                 void *workspace, const lrqk_peer_group *g, int32_t seq, lrqk_stream_t stream) {
  using namespace lrqk;
  if (!L) return LRQK_EINVAL;
  const int32_t rows = L->k + L->m;
  int rc = check_attn_args(L, q, out, rows);
  if (rc != LRQK_OK) return rc;
  if (!workspace || !mask || !L->table || !L->host_kv || L->host_capacity <= 0) return LRQK_EINVAL;
  if (g) {
    if (seq < 1) return LRQK_EINVAL;
    rc = check_peer_group(g);
    if (rc != LRQK_OK) return rc;
    if (g->heads_per_rank != L->bsz * L->q_heads || g->head_dim != L->head_dim || g->dtype != L->dtype) return LRQK_EINVAL;
  } else if (!out) {
    return LRQK_EINVAL;
  }
  return launch_flash_decode(L, q, out, rows, scale, workspace, as_stream(stream), g, seq, mask);
}

// ---------------------------------------------------------------------------------------------
// Attention without any allocation by anyone: the split partials and tickets live in an array
// that is part of the library image.
//
// Meant for callers that hold no allocator they may use at the time of the call: a plugin hook of
// a serving runtime that has already handed every byte of device memory to its own block pool, a
// latency-critical loop whose rules forbid allocator calls, an embedding host that only passes
// the input and output buffers through.  Such callers cannot size and provide the workspace
// lrqk_flash_decode() asks for, and this library must not call cudaMalloc on their behalf.
//
// The array is a file-scope __device__ object, so every GPU that loads the library carries it
// (kStaticScratchBytes) until the process exits.  In host code its name is only a handle; the
// address a kernel can use is obtained once per device with cudaGetSymbolAddress, while that
// device is current, and cached.
// ---------------------------------------------------------------------------------------------
namespace lrqk {
namespace {
constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB: e.g. 470 heads of head_dim 128 at 2112 bf16 rows (17 splits)
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticScratchBytes];
static void *g_static_scratch_ptr[lrqk::kMaxDevices] = {};  // device-usable address, per device
static int g_static_last_heads[lrqk::kMaxDevices] = {};      // head count of the last call: where its status word sits
}  // namespace
}  // namespace lrqk

extern "C" size_t lrqk_flash_decode_static_capacity_bytes(void) { return lrqk::kStaticScratchBytes; }

extern "C" int lrqk_flash_decode_static(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale,
                                        lrqk_stream_t stream) {
  using namespace lrqk;
  const int rc = check_attn_args(L, q, out, rows);
  if (rc != LRQK_OK) return rc;
  if (!out) return LRQK_EINVAL;
  const int n_heads = L->bsz * L->q_heads;
  const int splits = plan_splits((int)(L->head_dim * elt_size(L->dtype)), rows);
  const size_t ticket_bytes = ticket_region_bytes(n_heads);
  const size_t need = ticket_bytes + (size_t)n_heads * splits * (size_t)(L->head_dim + 2) * sizeof(float);
  if (need > kStaticScratchBytes) {
    char msg[200];
    snprintf(msg, sizeof(msg),
             "lrqk_flash_decode_static: %d heads x %d splits need %zu bytes of scratch, the built-in array holds %zu; "
             "use lrqk_flash_decode with a caller-provided workspace",
             n_heads, splits, need, kStaticScratchBytes);
    note_error_text(msg);
    return LRQK_ECAPACITY;
  }
  int dev = -1;
  LRQK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= lrqk::kMaxDevices) return LRQK_EUNSUPPORTED;
  if (!g_static_scratch_ptr[dev]) {  // set-up, once per device, with that device current
    void *ptr = nullptr;
    LRQK_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_attn_scratch));
    g_static_scratch_ptr[dev] = ptr;
  }
  char *scratch = reinterpret_cast<char *>(g_static_scratch_ptr[dev]);
  cudaStream_t s = as_stream(stream);
  // the array keeps whatever the previous call left: the tickets and the status word must start at zero
  LRQK_CUDA_TRY(cudaMemsetAsync(scratch, 0, ticket_bytes, s));
  g_static_last_heads[dev] = n_heads;
  return launch_flash_decode(L, q, out, rows, scale, scratch, s);
}

extern "C" int lrqk_flash_decode_static_status(int32_t *status_out, lrqk_stream_t stream) {
  using namespace lrqk;
  if (!status_out) return LRQK_EINVAL;
  int dev = -1;
  LRQK_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= lrqk::kMaxDevices) return LRQK_EUNSUPPORTED;
  if (!g_static_scratch_ptr[dev]) {  // no call on this device yet: nothing to report
    *status_out = 0;
    return LRQK_OK;
  }
  const int32_t *word = reinterpret_cast<const int32_t *>(g_static_scratch_ptr[dev]) + g_static_last_heads[dev];
  LRQK_CUDA_TRY(cudaMemcpyAsync(status_out, word, sizeof(int32_t), cudaMemcpyDeviceToHost, as_stream(stream)));
  return LRQK_OK;
}

extern "C" int32_t *lrqk_flash_decode_status_word(const lrqk_layer *L, void *workspace) {
  if (!L || !workspace || L->bsz <= 0 || L->q_heads <= 0) return nullptr;
  return reinterpret_cast<int32_t *>(workspace) + (size_t)L->bsz * L->q_heads;
}
