// Exact single-query attention over the resident rows, split over the row axis.
//
// Grid (splits, B*Hq).  A CTA streams its slice of K_res and V_res once with 16-byte loads
// (a K or V row is spread over d*elt/16 lanes), keeps a running (max, sum, accumulator) per
// lane group in fp32 with base-2 exponentials, and leaves one partial per split in the
// workspace.  The CTA that finishes last for a head (an atomic ticket) folds the partials in
// split order and writes the output row, then re-arms the ticket.
#include <math.h>
#include <stdio.h>

#include "common.cuh"

namespace lrqk {
namespace {

constexpr int kAThreads = 128;
constexpr int kAUnroll = 4;
constexpr int kMaxSplits = 32;

struct AttnParams {
  const void *q, *K_res, *V_res;
  void *out;
  float *partial;     // [N][splits][D+2]
  int32_t *tickets;   // [N]
  int32_t slots;      // rows allocated per head (k + m)
  int32_t rows;       // rows attended
  int32_t splits, chunk;
  float scale_log2;   // softmax scale * log2(e)
};

template <int EPV>
__device__ __forceinline__ void merge_state(float &m, float &l, float (&acc)[EPV], float m2, float l2,
                                            const float (&acc2)[EPV]) {
  const float mn = fmaxf(m, m2);
  if (mn == -INFINITY) return;  // both empty
  const float c1 = exp2f(m - mn), c2 = exp2f(m2 - mn);
  l = l * c1 + l2 * c2;
#pragma unroll
  for (int e = 0; e < EPV; ++e) acc[e] = acc[e] * c1 + acc2[e] * c2;
  m = mn;
}

template <typename T, int D>
__global__ void __launch_bounds__(kAThreads) flash_decode_kernel(AttnParams p) {
  constexpr int EPV = Elt<T>::kPerVec;            // elements per 16-byte vector
  constexpr int LPR = D / EPV;                    // lanes per row
  constexpr int GPW = 32 / LPR;                   // rows handled side by side in a warp
  constexpr int NWARP = kAThreads / 32;
  const int split = blockIdx.x, n = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int lir = lane % LPR, grp = lane / LPR;

  __shared__ float sm_acc[NWARP][LPR][EPV + 2];
  __shared__ int is_last;

  float qf[EPV];
  {
    float raw[EPV];
    Elt<T>::unpack(ld16(reinterpret_cast<const T *>(p.q) + (int64_t)n * D + lir * EPV), raw);
#pragma unroll
    for (int e = 0; e < EPV; ++e) qf[e] = raw[e] * p.scale_log2;
  }
  const T *Kb = reinterpret_cast<const T *>(p.K_res) + (int64_t)n * p.slots * D + lir * EPV;
  const T *Vb = reinterpret_cast<const T *>(p.V_res) + (int64_t)n * p.slots * D + lir * EPV;
  const int r_begin = split * p.chunk;
  const int r_end = min(p.rows, r_begin + p.chunk);

  float m_run = -INFINITY, l_run = 0.0f, acc[EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) acc[e] = 0.0f;

  constexpr int STEP = NWARP * GPW;  // rows per CTA-wide load
  for (int base = r_begin; base < r_end; base += kAUnroll * STEP) {  // CTA-uniform trip count
    const int r0 = base + warp * GPW + grp;
    uint4 kv[kAUnroll], vv[kAUnroll];
#pragma unroll
    for (int u = 0; u < kAUnroll; ++u) {
      const int row = r0 + u * STEP;
      if (row < r_end) {
        kv[u] = ld16(Kb + (int64_t)row * D);
        vv[u] = ld16(Vb + (int64_t)row * D);
      }
    }
#pragma unroll
    for (int u = 0; u < kAUnroll; ++u) {
      const int row = r0 + u * STEP;
      const bool valid = row < r_end;
      float kf[EPV], vf[EPV];
      float s = 0.0f;
      if (valid) {
        Elt<T>::unpack(kv[u], kf);
        Elt<T>::unpack(vv[u], vf);
#pragma unroll
        for (int e = 0; e < EPV; ++e) s = fmaf(kf[e], qf[e], s);
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, o);
      if (valid) {
        const float mn = fmaxf(m_run, s);
        const float corr = exp2f(m_run - mn);  // exp2f(-inf) = 0 on the first row
        const float pr = exp2f(s - mn);
        l_run = l_run * corr + pr;
#pragma unroll
        for (int e = 0; e < EPV; ++e) acc[e] = acc[e] * corr + pr * vf[e];
        m_run = mn;
      }
    }
  }
  // fold the row groups of a warp, then the warps of the CTA
#pragma unroll
  for (int o = LPR; o < 32; o <<= 1) {
    const float m2 = __shfl_xor_sync(0xFFFFFFFFu, m_run, o);
    const float l2 = __shfl_xor_sync(0xFFFFFFFFu, l_run, o);
    float a2[EPV];
#pragma unroll
    for (int e = 0; e < EPV; ++e) a2[e] = __shfl_xor_sync(0xFFFFFFFFu, acc[e], o);
    merge_state<EPV>(m_run, l_run, acc, m2, l2, a2);
  }
  if (grp == 0) {
#pragma unroll
    for (int e = 0; e < EPV; ++e) sm_acc[warp][lir][e] = acc[e];
    sm_acc[warp][lir][EPV] = m_run;
    sm_acc[warp][lir][EPV + 1] = l_run;
  }
  __syncthreads();
  float *part = p.partial + ((int64_t)n * p.splits + split) * (D + 2);
  if (warp == 0 && grp == 0) {
#pragma unroll
    for (int w = 1; w < NWARP; ++w) {
      float a2[EPV];
#pragma unroll
      for (int e = 0; e < EPV; ++e) a2[e] = sm_acc[w][lir][e];
      merge_state<EPV>(m_run, l_run, acc, sm_acc[w][lir][EPV], sm_acc[w][lir][EPV + 1], a2);
    }
#pragma unroll
    for (int e = 0; e < EPV; ++e) part[lir * EPV + e] = acc[e];
    if (lir == 0) { part[D] = m_run; part[D + 1] = l_run; }
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
  // fold the partials of this head in split order
  const float *ph = p.partial + (int64_t)n * p.splits * (D + 2);
  float mx = -INFINITY;
  for (int s = 0; s < p.splits; ++s) mx = fmaxf(mx, __ldcg(ph + (int64_t)s * (D + 2) + D));
  for (int e = tid; e < D; e += kAThreads) {
    float num = 0.0f, den = 0.0f;
    for (int s = 0; s < p.splits; ++s) {
      const float *ps = ph + (int64_t)s * (D + 2);
      const float ms = __ldcg(ps + D);
      if (ms == -INFINITY) continue;
      const float c = exp2f(ms - mx);
      num = fmaf(__ldcg(ps + e), c, num);
      den = fmaf(__ldcg(ps + D + 1), c, den);
    }
    reinterpret_cast<T *>(p.out)[(int64_t)n * D + e] = Elt<T>::from_float(num / den);
  }
  if (tid == 0) p.tickets[n] = 0;  // re-arm for the next call
}

int plan_splits(int n_heads, int rows) {
  int splits = (4 * kNumSMs + n_heads - 1) / n_heads;
  if (splits > kMaxSplits) splits = kMaxSplits;
  const int by_rows = rows / 32;
  if (splits > by_rows) splits = by_rows;
  if (splits < 1) splits = 1;
  return splits;
}

}  // namespace
}  // namespace lrqk

extern "C" size_t lrqk_flash_decode_workspace_bytes(const lrqk_layer *L, int32_t rows) {
  (void)rows;
  if (!L) return 0;
  const size_t n = (size_t)L->bsz * L->q_heads;
  return n * sizeof(int32_t) + 256 + n * lrqk::kMaxSplits * (size_t)(L->head_dim + 2) * sizeof(float);
}

extern "C" int lrqk_flash_decode(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale,
                                 void *workspace, lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!q || !out || !workspace || !L->K_res || !L->V_res) return LRQK_EINVAL;
  if (rows <= 0) return LRQK_EINVAL;
  if (rows > L->k + L->m) return LRQK_ECAPACITY;
  const int n_heads = L->bsz * L->q_heads;
  if (n_heads > 65535) return LRQK_EUNSUPPORTED;
  AttnParams p;
  p.q = q; p.K_res = L->K_res; p.V_res = L->V_res; p.out = out;
  p.tickets = reinterpret_cast<int32_t *>(workspace);
  const size_t off = ((size_t)n_heads * sizeof(int32_t) + 255) / 256 * 256;
  p.partial = reinterpret_cast<float *>(reinterpret_cast<char *>(workspace) + off);
  p.slots = L->k + L->m;
  p.rows = rows;
  p.splits = plan_splits(n_heads, rows);
  p.chunk = (rows + p.splits - 1) / p.splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(p.splits, n_heads, 1);
  cudaStream_t s = as_stream(stream);
  if (L->head_dim == 128) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, (flash_decode_kernel<T, 128><<<grid, kAThreads, 0, s>>>(p)));
  } else if (L->head_dim == 64) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, (flash_decode_kernel<T, 64><<<grid, kAThreads, 0, s>>>(p)));
  } else {
    return LRQK_EUNSUPPORTED;
  }
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
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
constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB: up to 240 heads of head_dim 128
constexpr int kMaxDevices = 64;
static __device__ __align__(256) unsigned char g_static_attn_scratch[kStaticScratchBytes];
static void *g_static_scratch_ptr[kMaxDevices] = {};  // device-usable address, per device
}  // namespace
}  // namespace lrqk

extern "C" size_t lrqk_flash_decode_static_capacity_bytes(void) { return lrqk::kStaticScratchBytes; }

extern "C" int lrqk_flash_decode_static(const lrqk_layer *L, const void *q, void *out, int32_t rows, float scale,
                                        lrqk_stream_t stream) {
  using namespace lrqk;
  int rc = check_device();
  if (rc != LRQK_OK) return rc;
  rc = check_layer(L);
  if (rc != LRQK_OK) return rc;
  if (!q || !out || !L->K_res || !L->V_res) return LRQK_EINVAL;
  if (rows <= 0) return LRQK_EINVAL;
  if (rows > L->k + L->m) return LRQK_ECAPACITY;
  const int n_heads = L->bsz * L->q_heads;
  if (n_heads > 65535) return LRQK_EUNSUPPORTED;
  if (L->head_dim != 128 && L->head_dim != 64) return LRQK_EUNSUPPORTED;
  const int splits = plan_splits(n_heads, rows);
  const size_t ticket_bytes = ((size_t)n_heads * sizeof(int32_t) + 255) / 256 * 256;
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
  if (dev < 0 || dev >= kMaxDevices) return LRQK_EUNSUPPORTED;
  if (!g_static_scratch_ptr[dev]) {  // set-up, once per device, with that device current
    void *ptr = nullptr;
    LRQK_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_attn_scratch));
    g_static_scratch_ptr[dev] = ptr;
  }
  char *scratch = reinterpret_cast<char *>(g_static_scratch_ptr[dev]);
  cudaStream_t s = as_stream(stream);
  // the array keeps whatever the previous call left: the tickets must start at zero
  LRQK_CUDA_TRY(cudaMemsetAsync(scratch, 0, ticket_bytes, s));
  AttnParams p;
  p.q = q; p.K_res = L->K_res; p.V_res = L->V_res; p.out = out;
  p.tickets = reinterpret_cast<int32_t *>(scratch);
  p.partial = reinterpret_cast<float *>(scratch + ticket_bytes);
  p.slots = L->k + L->m;
  p.rows = rows;
  p.splits = splits;
  p.chunk = (rows + splits - 1) / splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  dim3 grid(splits, n_heads, 1);
  if (L->head_dim == 128) {
    LRQK_DISPATCH_DTYPE(L->dtype, T, (flash_decode_kernel<T, 128><<<grid, kAThreads, 0, s>>>(p)));
  } else {
    LRQK_DISPATCH_DTYPE(L->dtype, T, (flash_decode_kernel<T, 64><<<grid, kAThreads, 0, s>>>(p)));
  }
  LRQK_LAUNCH_CHECK();
  return LRQK_OK;
}
