// Apply pass of the prompt factorisation on the tensor cores:  A_K[head] = K[kv head] X_K[head]
// for every prompt row, bf16 prompts with head_dim 128.
//
// One CTA handles a run of 128-row prompt tiles of one (batch, KV head) and up to 128/r of the
// query heads that share it: their X_K matrices (d x r, fp32, the sweep chosen by the stop test)
// are split into a high and a low bf16 part and laid side by side as the B operand (N = heads * r
// rows of 128 K-major elements, 128-byte swizzle), so a K tile is read once for all of them.  A tile
// is two TMA tensor copies of [128 rows][64 dims]; sixteen tcgen05 MMAs (M128, N, K16: eight K steps
// times the two parts of X_K) form the tile's product in one
// of two TMEM accumulators, and four epilogue warps turn the other accumulator into bf16 rows of
// A_K meanwhile.  Warp 0 issues copies, warp 1 owns TMEM and issues MMAs, warps 2-5 prepare B and
// run the epilogue.  Every wait is bounded (status word, TMEM freed on the way out).
#include "apply_tc.cuh"
#include "tc_common.cuh"

namespace lrqk {
namespace {

using namespace tc;

constexpr int kATileRows = 128;
constexpr int kABlockBytes = kATileRows * 128;      // [128 rows][64 dims] bf16
constexpr int kAStageBytes = 2 * kABlockBytes;      // both halves of the 128 dims
constexpr int kAStages = 4;
constexpr int kAThreadsTc = 192;
constexpr int kMaxN = 128;                          // columns of one accumulator (query heads of a CTA times r)
constexpr int kBPartBytes = 2 * kMaxN * 128;        // one bf16 part of B: 2 blocks of [kMaxN rows][128 bytes]

struct ApplyTcParams {
  const float *ws;        // workspace of the factorisation (per-sweep results)
  void *A_K;              // [B*Hq][a_capacity][R] bf16
  int32_t *status;
  int64_t seq_len, a_capacity, sweep_base;
  int32_t sweep_stride, sweeps, n_heads, q_heads, groups, heads_per_cta, chunks, tiles_per_cta;
  float tol;
};

template <int R>
__global__ void __launch_bounds__(kAThreadsTc, 1) apply_tc_kernel(const __grid_constant__ CUtensorMap mapK, ApplyTcParams p) {
  constexpr int D = 128;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int unit = blockIdx.y / p.chunks, chunk = blockIdx.y % p.chunks;   // unit = b * Hkv + kvh
  const int kv_heads = p.q_heads / p.groups;
  const int b = unit / kv_heads, kvh = unit % kv_heads;
  const int g0 = chunk * p.heads_per_cta;
  const int n_g = min(p.heads_per_cta, p.groups - g0);     // query heads of this CTA
  const int N = (n_g * R + 15) / 16 * 16;                  // MMA N (zero rows pad it to a multiple of 16)
  const int head0 = b * p.q_heads + kvh * p.groups + g0;   // first query head (index into [B*Hq])

  extern __shared__ unsigned char smem_raw[];
  unsigned char *stages = smem_raw + ((1024u - (saddr(smem_raw) & 1023u)) & 1023u);
  unsigned char *Bsm = stages + (size_t)kAStages * kAStageBytes;        // X_K as two bf16 parts (high, low)
  uint64_t *bars = reinterpret_cast<uint64_t *>(Bsm + 2 * kBPartBytes);
  uint64_t *full = bars, *empty = bars + kAStages, *acc_full = bars + 2 * kAStages, *acc_empty = acc_full + 2;
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_empty + 2);
  volatile int *give_up = reinterpret_cast<volatile int *>(tmem_slot + 1);
  int *chosen_p = const_cast<int *>(give_up) + 1;
  float *delta = reinterpret_cast<float *>(chosen_p + 1);  // [2][8]

  const int tile0 = blockIdx.x * p.tiles_per_cta;
  const int total_tiles = (int)((p.seq_len + kATileRows - 1) / kATileRows);
  const int n_tiles = max(0, min(p.tiles_per_cta, total_tiles - tile0));
  const uint32_t tmem_cols = N <= 16 ? 32u : (N <= 32 ? 64u : (N <= 64 ? 128u : 256u));
  const uint32_t acc_stride = tmem_cols / 2;

  if (tid == 0) {
    for (int s = 0; s < kAStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
    *give_up = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // stopping sweep: first sweep whose mean squared change of both left factors is below tol
  // (a mean over ALL heads, as in the reference; every CTA derives the same value)
  for (int i = warp; i < 2 * p.sweeps; i += kAThreadsTc / 32) {
    const int sw = i >> 1, which = i & 1;
    float s = 0.0f;
    for (int hh = lane; hh < p.n_heads; hh += 32)
      s += p.ws[p.sweep_base + ((int64_t)hh * p.sweeps + sw) * p.sweep_stride + 4 * R * D + which];
    s = warp_sum(s);
    if (lane == 0) delta[which * 8 + sw] = s / ((float)p.n_heads * (float)p.seq_len * (float)R);
  }
  __syncthreads();
  if (tid == 0) {
    int c = p.sweeps - 1;
    for (int sw = 0; sw < p.sweeps; ++sw)
      if (fmaxf(delta[sw], delta[8 + sw]) < p.tol) { c = sw; break; }
    *chosen_p = c;
  }
  __syncthreads();
  const int chosen = *chosen_p;
  // B operand: row (g, c) of block e/64 holds X_K[head g][e][c] for e = 0..127.  X_K is fp32; it
  // enters as the sum of two bf16 parts (x = hi + lo, lo = bf16(x - hi)), each multiplied into the
  // same accumulator, so the product keeps ~16 mantissa bits of X_K: rounding it to one bf16 would
  // add as much error to A_K as the final rounding of A_K itself.
  for (int i = tid; i < 2 * kBPartBytes / 16; i += kAThreadsTc) reinterpret_cast<uint4 *>(Bsm)[i] = make_uint4(0, 0, 0, 0);
  __syncthreads();
  for (int i = tid; i < n_g * R * D; i += kAThreadsTc) {
    const int g = i / (R * D), rem = i % (R * D), e = rem / R, c = rem % R;   // consecutive threads: consecutive c
    const float x = p.ws[p.sweep_base + ((int64_t)(head0 + g) * p.sweeps + chosen) * p.sweep_stride + D * R + e * R + c];
    const int row = g * R + c, blk = e >> 6, chunk16 = (e & 63) >> 3;
    const size_t at = (size_t)blk * kMaxN * 128 + row * 128 + ((chunk16 ^ (row & 7)) << 4) + (e & 7) * 2;
    const __nv_bfloat16 hi = __float2bfloat16_rn(x);
    *reinterpret_cast<__nv_bfloat16 *>(Bsm + at) = hi;
    *reinterpret_cast<__nv_bfloat16 *>(Bsm + kBPartBytes + at) = __float2bfloat16_rn(x - __bfloat162float(hi));
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int t = 0; t < n_tiles && !*give_up; ++t) {
        const int s = t % kAStages;
        if (t >= kAStages && !wait_bounded(&empty[s], ((t / kAStages) - 1) & 1)) { *give_up = 1; atomicExch(p.status, (int32_t)LRQK_ETIMEOUT); break; }
        unsigned char *st = stages + (size_t)s * kAStageBytes;
        const int row0 = (tile0 + t) * kATileRows;
        mbar_expect_tx(&full[s], kAStageBytes);
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                     ::"r"(saddr(st)), "l"(&mapK), "r"(saddr(&full[s])), "r"(0), "r"(row0), "r"(unit) : "memory");
        asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                     ::"r"(saddr(st + kABlockBytes)), "l"(&mapK), "r"(saddr(&full[s])), "r"(64), "r"(row0), "r"(unit) : "memory");
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16_k(128, N);
      const uint32_t b_base = saddr(Bsm);
      for (int t = 0; t < n_tiles && !*give_up; ++t) {
        const int s = t % kAStages, a = t & 1;
        if (!wait_bounded(&full[s], (t / kAStages) & 1) ||
            (t >= 2 && !wait_bounded(&acc_empty[a], ((t >> 1) - 1) & 1))) { *give_up = 1; atomicExch(p.status, (int32_t)LRQK_ETIMEOUT); break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_base = saddr(stages + (size_t)s * kAStageBytes);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t blk = ks >> 2, off = (ks & 3) * 32;
          const uint64_t adesc = umma_desc_k_sw128(a_base + blk * kABlockBytes + off, 1024);
          umma_bf16(tmem_base + a * acc_stride, adesc, umma_desc_k_sw128(b_base + blk * (kMaxN * 128) + off, 1024), idesc,
                    ks > 0 ? 1u : 0u);
          umma_bf16(tmem_base + a * acc_stride, adesc,
                    umma_desc_k_sw128(b_base + kBPartBytes + blk * (kMaxN * 128) + off, 1024), idesc, 1u);
        }
        umma_commit(&empty[s]);
        umma_commit(&acc_full[a]);
      }
    }
  } else {
    // ---- epilogue warps: accumulator -> bf16 rows of A_K ---------------------------------------------
    const int quarter = warp & 3, row_in_tile = quarter * 32 + lane;
    __nv_bfloat16 *AK = reinterpret_cast<__nv_bfloat16 *>(p.A_K);
    for (int t = 0; t < n_tiles && !*give_up; ++t) {
      const int a = t & 1;
      if (!wait_bounded(&acc_full[a], (t >> 1) & 1)) { *give_up = 1; atomicExch(p.status, (int32_t)LRQK_ETIMEOUT); break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int64_t row = (int64_t)(tile0 + t) * kATileRows + row_in_tile;
      const uint32_t taddr = tmem_base + a * acc_stride + ((uint32_t)(quarter * 32) << 16);
      for (int g = 0; g < n_g; ++g) {
#pragma unroll
        for (int c0 = 0; c0 < R; c0 += 32) {
          uint32_t v[32];
          if constexpr (R >= 32) tmem_ld32(taddr + g * R + c0, v);
          else if constexpr (R == 16) tmem_ld16(taddr + g * R + c0, v);
          else tmem_ld8(taddr + g * R + c0, v);
          if (row < p.seq_len) {
            __nv_bfloat16 *dst = AK + ((int64_t)(head0 + g) * p.a_capacity + row) * R + c0;
            constexpr int CW = R < 32 ? R : 32;
#pragma unroll
            for (int j = 0; j < CW; j += 8) {
              uint4 pk;
              __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(v[j]), __uint_as_float(v[j + 1]));
              __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
              __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
              __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
              pk.x = *reinterpret_cast<uint32_t *>(&h0); pk.y = *reinterpret_cast<uint32_t *>(&h1);
              pk.z = *reinterpret_cast<uint32_t *>(&h2); pk.w = *reinterpret_cast<uint32_t *>(&h3);
              *reinterpret_cast<uint4 *>(dst + j) = pk;
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(&acc_empty[a]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

template <int R>
int launch_r(const ApplyTcArgs &a, cudaStream_t stream) {
  constexpr size_t smem = (size_t)kAStages * kAStageBytes + 2 * kBPartBytes + (2 * kAStages + 4) * 8 + 16 + 16 * 4 + 1024;
  auto kern = apply_tc_kernel<R>;
  static SmemOptIn opt_in;
  LRQK_CUDA_TRY(opt_in.ensure(kern, smem));
  CUtensorMap mk;
  const int rc = make_prompt_map(&mk, a.K, (int64_t)a.bsz * a.kv_heads, a.seq_len, kATileRows);
  if (rc != LRQK_OK) return rc;
  ApplyTcParams p;
  p.ws = a.ws; p.A_K = a.A_K; p.status = a.status;
  p.seq_len = a.seq_len; p.a_capacity = a.a_capacity; p.sweep_base = a.sweep_base;
  p.sweep_stride = a.sweep_stride; p.sweeps = a.sweeps; p.n_heads = a.bsz * a.q_heads; p.q_heads = a.q_heads;
  p.groups = a.q_heads / a.kv_heads;
  p.heads_per_cta = kMaxN / (R < 16 ? 16 : R);   // N stays a multiple of 16 and at most kMaxN
  if (p.heads_per_cta > p.groups) p.heads_per_cta = p.groups;
  p.chunks = (p.groups + p.heads_per_cta - 1) / p.heads_per_cta;
  p.tol = a.tol;
  const int total_tiles = (int)ceil_div64(a.seq_len, kATileRows);
  // enough CTAs for a few waves, each with a run of tiles long enough to amortise its set-up
  const int units = a.bsz * a.kv_heads * p.chunks;
  int per = (int)ceil_div64((int64_t)total_tiles * units, 4 * kNumSMs);
  if (per < 4) per = 4;
  p.tiles_per_cta = per;
  const unsigned gx = (unsigned)ceil_div64(total_tiles, per);
  if (units > 65535) return LRQK_EUNSUPPORTED;
  kern<<<dim3(gx, units, 1), kAThreadsTc, smem, stream>>>(mk, p);
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}

}  // namespace

int launch_apply_tc(const ApplyTcArgs &a, cudaStream_t stream) {
  if (a.head_dim != 128) return LRQK_EUNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(a.K) | reinterpret_cast<uintptr_t>(a.A_K)) & 15) return LRQK_EUNSUPPORTED;
  if (a.seq_len >= (1ll << 31) || a.sweeps > 8) return LRQK_EUNSUPPORTED;
  switch (a.r) {
    case 8: return launch_r<8>(a, stream);
    case 16: return launch_r<16>(a, stream);
    case 32: return launch_r<32>(a, stream);
    case 64: return launch_r<64>(a, stream);
    default: return LRQK_EUNSUPPORTED;
  }
}

}  // namespace lrqk
