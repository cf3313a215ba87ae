// Gram pass of the prompt factorisation on the 5th-generation tensor cores (tcgen05 + TMEM),
// fed by TMA.  bf16 prompts with head_dim 128.
//
// Per (head, side, split) one CTA accumulates, over its rows of the prompt,
//     D1 = X^T [X | A0]      (128 x 192, the last 64 columns hold A0 padded with zeros)
//     D2 = [X_hi | A0]^T A0  (128 x 64; rows 64.. are A0^T A0)
// where X is the head's Q (side 0) or K (side 1) and A0 the initial left factor.  Both products
// contract over the prompt rows, and X is stored row-major [row][dim]: the contraction index is
// the slow one, so both operands are "MN-major" for the tensor core and one shared-memory tile
// serves as A and as B.
//
// Shared-memory stage (64 prompt rows): three 64-column groups, each [64 rows][128 bytes] in the
// 128-byte swizzle -- X[:, 0:64] and X[:, 64:128] written by two TMA tensor copies, and A0
// (fp32 in memory) rounded to bf16 and zero-padded to 64 columns by four converter warps, which
// read the fp32 rows from a staging area that a bulk copy fills.  An MMA covers 16 rows, so a
// stage is four steps of two instructions (M128 N192 K16 and M128 N64 K16).
//
// Warp roles: warp 0 issues the copies, warp 1 owns TMEM and issues the MMAs, warps 2-5 convert
// A0 and, at the end, read the accumulators from TMEM and write the partial Gram block of this
// split in the layout the algebra kernel sums.  Stages are recycled through mbarriers; the MMA
// warp releases a stage with tcgen05.commit.  Every wait is bounded: if one runs out the CTA
// raises the status word, stops issuing work, and still frees its TMEM.
#include "common.cuh"
#include "gram_tc.cuh"
#include "tc_common.cuh"

namespace lrqk {
namespace {

using namespace tc;

constexpr int kTileRows = 64;                       // prompt rows per stage
constexpr int kGroupBytes = kTileRows * 128;        // one 64-column group of a stage
template <int R> __host__ __device__ constexpr int stage_count() { return R >= 64 ? 5 : 6; }  // 160 to 200 KiB of stages
constexpr int kTcThreads = 192;                     // 6 warps
constexpr int kTmemCols = 256;

struct GramTcParams {
  const float *A_Q0, *A_K0;   // [N][S][R] fp32
  float *part;                // [2][N][splits][Wp*Wp]
  int32_t *status;
  int64_t seq_len;
  int32_t q_heads, groups, splits, rows_per_split, n_heads;
};

template <int R>
__global__ void __launch_bounds__(kTcThreads, 1) gram_tc_kernel(const __grid_constant__ CUtensorMap mapQ,
                                                               const __grid_constant__ CUtensorMap mapK, GramTcParams p) {
  constexpr int D = 128, W = R + D, Wp = (W + 15) / 16 * 16;
  constexpr int kRawBytes = kTileRows * R * 4;                 // fp32 A0 rows of a stage
  constexpr int kStageBytes = 3 * kGroupBytes + kRawBytes;
  constexpr int kStages = stage_count<R>();
  constexpr uint32_t kIdesc1 = umma_idesc_bf16_mn(128, 192), kIdesc2 = umma_idesc_bf16_mn(128, 64);

  const int split = blockIdx.x, n = blockIdx.y, side = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = n / p.q_heads, h = n % p.q_heads, kv_heads = p.q_heads / p.groups;
  const int x_head = side == 0 ? n : b * kv_heads + h / p.groups;  // which [S][128] slab of the tensor map
  const float *A0 = (side == 0 ? p.A_Q0 : p.A_K0) + (int64_t)n * p.seq_len * R;

  extern __shared__ unsigned char smem_raw[];
  // kStages x {group 0, group 1, group 2, raw fp32 A0}; the swizzle needs 1024-byte aligned stages
  unsigned char *stages = smem_raw + ((1024u - (saddr(smem_raw) & 1023u)) & 1023u);
  uint64_t *bars = reinterpret_cast<uint64_t *>(stages + (size_t)kStages * kStageBytes);
  uint64_t *full = bars;                  // [kStages] copies of the stage have landed
  uint64_t *conv = bars + kStages;        // [kStages] A0 of the stage is converted
  uint64_t *empty = bars + 2 * kStages;   // [kStages] the MMAs that read the stage have retired
  uint64_t *acc_done = bars + 3 * kStages;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * kStages + 1);
  volatile int *give_up = reinterpret_cast<volatile int *>(tmem_slot + 1);

  const int64_t r_begin = (int64_t)split * p.rows_per_split;
  const int64_t r_end = min(p.seq_len, r_begin + p.rows_per_split);
  const int n_tiles = r_end > r_begin ? (int)((r_end - r_begin + kTileRows - 1) / kTileRows) : 0;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&conv[s], 128);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_done, 1);
    *give_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // the padding columns of group 2 never change: clear every stage's group 2 once
  for (int i = tid; i < kStages * kGroupBytes / 16; i += kTcThreads) {
    const int s = i / (kGroupBytes / 16), o = i % (kGroupBytes / 16);
    *reinterpret_cast<uint4 *>(stages + (size_t)s * kStageBytes + 2 * kGroupBytes + (size_t)o * 16) = make_uint4(0, 0, 0, 0);
  }
  if (warp == 1) {  // TMEM: 256 columns (192 for D1, 64 for D2)
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(tmem_slot)), "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the zero fill above is read by the tensor core
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---- producer: one lane issues the copies of every stage ---------------------------------
    if (lane == 0) {
      const CUtensorMap *map = side == 0 ? &mapQ : &mapK;
      for (int t = 0; t < n_tiles && !*give_up; ++t) {
        const int s = t % kStages;
        if (t >= kStages && !wait_bounded(&empty[s], ((t / kStages) - 1) & 1)) { *give_up = 1; atomicExch(p.status, (int32_t)LRQK_ETIMEOUT); break; }
        unsigned char *st = stages + (size_t)s * kStageBytes;
        const int64_t row0 = r_begin + (int64_t)t * kTileRows;
        const int rows = (int)min((int64_t)kTileRows, r_end - row0);
        const uint32_t raw_bytes = (uint32_t)rows * R * 4;
        mbar_expect_tx(&full[s], 2 * kGroupBytes + raw_bytes);
        // rows past the end of the prompt are filled with zeros by the tensor copy
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                     ::"r"(saddr(st)), "l"(map), "r"(saddr(&full[s])), "r"(0), "r"((int)row0), "r"(x_head) : "memory");
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                     ::"r"(saddr(st + kGroupBytes)), "l"(map), "r"(saddr(&full[s])), "r"(64), "r"((int)row0), "r"(x_head) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                     ::"r"(saddr(st + 3 * kGroupBytes)), "l"(A0 + row0 * R), "r"(raw_bytes), "r"(saddr(&full[s])) : "memory");
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer -----------------------------------------------------------------------------
    if (lane == 0) {
      for (int t = 0; t < n_tiles && !*give_up; ++t) {
        const int s = t % kStages;
        const uint32_t ph = (t / kStages) & 1;
        if (!wait_bounded(&full[s], ph) || !wait_bounded(&conv[s], ph)) { *give_up = 1; atomicExch(p.status, (int32_t)LRQK_ETIMEOUT); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t base = saddr(stages + (size_t)s * kStageBytes);
#pragma unroll
        for (int ks = 0; ks < kTileRows / 16; ++ks) {
          const uint32_t off = ks * 2048;  // 16 rows of 128 bytes
          const uint32_t accumulate = (t > 0 || ks > 0) ? 1u : 0u;
          // D1 += X^T [X | A0]
          umma_bf16(tmem_base, umma_desc_mn_sw128(base + off, kGroupBytes, 1024),
                    umma_desc_mn_sw128(base + off, kGroupBytes, 1024), kIdesc1, accumulate);
          // D2 += [X_hi | A0]^T A0
          umma_bf16(tmem_base + 192, umma_desc_mn_sw128(base + kGroupBytes + off, kGroupBytes, 1024),
                    umma_desc_mn_sw128(base + 2 * kGroupBytes + off, kGroupBytes, 1024), kIdesc2, accumulate);
        }
        umma_commit(&empty[s]);  // arrives once the MMAs above have read the stage
      }
      umma_commit(acc_done);     // arrives once every MMA issued so far has completed
    }
  } else {
    // ---- converter warps: A0 fp32 -> bf16 into group 2, in the swizzled layout ---------------------
    const int ct = tid - 64;  // 0..127
    for (int t = 0; t < n_tiles && !*give_up; ++t) {
      const int s = t % kStages;
      if (!wait_bounded(&full[s], (t / kStages) & 1)) { *give_up = 1; atomicExch(p.status, (int32_t)LRQK_ETIMEOUT); break; }
      unsigned char *st = stages + (size_t)s * kStageBytes;
      const float4 *raw = reinterpret_cast<const float4 *>(st + 3 * kGroupBytes);
      unsigned char *g2 = st + 2 * kGroupBytes;
      const int64_t row0 = r_begin + (int64_t)t * kTileRows;
      const int rows = (int)min((int64_t)kTileRows, r_end - row0);
      constexpr int QPR = R / 4;  // float4 per row
      for (int i = ct; i < kTileRows * QPR; i += 128) {
        const int row = i / QPR, c4 = i % QPR;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < rows) v = raw[i];
        __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t *>(&lo);
        pk.y = *reinterpret_cast<uint32_t *>(&hi);
        const int chunk = c4 >> 1;  // 16-byte chunk of the 128-byte row
        *reinterpret_cast<uint2 *>(g2 + row * 128 + ((chunk ^ (row & 7)) << 4) + (c4 & 1) * 8) = pk;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
      mbar_arrive(&conv[s]);
    }
    // ---- epilogue: accumulators -> this split's partial Gram block -----------------------------------
    if (!*give_up && n_tiles > 0 && !wait_bounded(acc_done, 0)) { *give_up = 1; atomicExch(p.status, (int32_t)LRQK_ETIMEOUT); }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    float *out = p.part + ((((int64_t)side * p.n_heads + n) * p.splits) + split) * (int64_t)(Wp * Wp);
    const int quarter = warp & 3;          // the TMEM lanes a warp may read: 32 * (warp % 4) ...
    const int row = quarter * 32 + lane;   // row of D1 / D2 held by this thread
    const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const bool live = __shfl_sync(0xFFFFFFFFu, (!*give_up && n_tiles > 0) ? 1 : 0, 0) != 0;  // warp-uniform
    uint32_t v[32];
    for (int c0 = 0; c0 < 128; c0 += 32) {           // X^T X
      if (live) tmem_ld32(lane_addr + c0, v);
      else { for (int j = 0; j < 32; ++j) v[j] = 0u; }
      float4 *dst = reinterpret_cast<float4 *>(out + (int64_t)row * Wp + c0);
#pragma unroll
      for (int j = 0; j < 8; ++j) dst[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                       __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
    }
    for (int c0 = 0; c0 < R; c0 += 32) {             // (X^T A0)^T = A0^T X
      if (live) tmem_ld32(lane_addr + 128 + c0, v);
      else { for (int j = 0; j < 32; ++j) v[j] = 0u; }
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c0 + j < R) out[(int64_t)(D + c0 + j) * Wp + row] = __uint_as_float(v[j]);
    }
    for (int c0 = 0; c0 < R; c0 += 32) {             // A0^T A0: rows 64 .. 64 + R of D2
      if (live) tmem_ld32(lane_addr + 192 + c0, v);  // (every lane of the warp takes part in the load)
      else { for (int j = 0; j < 32; ++j) v[j] = 0u; }
      if (row >= 64 && row < 64 + R) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c0 + j < R) out[(int64_t)(D + row - 64) * Wp + D + c0 + j] = __uint_as_float(v[j]);
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

template <int R>
int launch_r(const GramTcArgs &a, cudaStream_t stream) {
  constexpr int kRawBytes = kTileRows * R * 4;
  constexpr int kStages = stage_count<R>();
  constexpr size_t smem = (size_t)kStages * (3 * kGroupBytes + kRawBytes) + (3 * kStages + 1) * 8 + 16 + 1024;
  auto kern = gram_tc_kernel<R>;
  static SmemOptIn opt_in;
  LRQK_CUDA_TRY(opt_in.ensure(kern, smem));
  CUtensorMap mq, mk;
  int rc = make_prompt_map(&mq, a.Q, (int64_t)a.bsz * a.q_heads, a.seq_len, kTileRows);
  if (rc != LRQK_OK) return rc;
  rc = make_prompt_map(&mk, a.K, (int64_t)a.bsz * a.kv_heads, a.seq_len, kTileRows);
  if (rc != LRQK_OK) return rc;
  GramTcParams p;
  p.A_Q0 = a.A_Q0; p.A_K0 = a.A_K0; p.part = a.part; p.status = a.status;
  p.seq_len = a.seq_len; p.q_heads = a.q_heads; p.groups = a.q_heads / a.kv_heads;
  p.splits = a.splits; p.rows_per_split = a.rows_per_split; p.n_heads = a.bsz * a.q_heads;
  kern<<<dim3(a.splits, a.bsz * a.q_heads, 2), kTcThreads, smem, stream>>>(mq, mk, p);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

}  // namespace

int gram_tc_tile_rows() { return kTileRows; }

int launch_gram_tc(const GramTcArgs &a, cudaStream_t stream) {
  if (a.head_dim != 128) return LRQK_EUNSUPPORTED;
  // the tensor copies need 16-byte aligned bases; the fp32 rows of A0 are copied in bulk
  if ((reinterpret_cast<uintptr_t>(a.Q) | reinterpret_cast<uintptr_t>(a.K) | reinterpret_cast<uintptr_t>(a.A_Q0) |
       reinterpret_cast<uintptr_t>(a.A_K0)) & 15)
    return LRQK_EUNSUPPORTED;
  if (a.rows_per_split % kTileRows != 0 || a.seq_len >= (1ll << 31)) return LRQK_EUNSUPPORTED;
  switch (a.r) {
    case 8: return launch_r<8>(a, stream);
    case 16: return launch_r<16>(a, stream);
    case 32: return launch_r<32>(a, stream);
    case 64: return launch_r<64>(a, stream);
    default: return LRQK_EUNSUPPORTED;
  }
}

}  // namespace lrqk
