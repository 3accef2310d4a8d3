// Routed feed-forward (mixture of experts): every token picks `top` of `experts` small gated feed-forward layers.
//
//  * route:   logits = h W_r^T in 32-bit (one warp per token, lanes stride the width, a fixed order of additions);
//             the `top` largest logits (the lower index wins a tie); weights = softmax over the chosen logits only;
//             optionally a gate for a shared expert, sigmoid(h . w_sg).
//  * plan:    a stable counting sort of the (token, choice) entries by expert, entirely on the device, so that a step
//             has the same launches whatever the tokens choose (it can be recorded and replayed): per segment of 1,024
//             entries each entry's rank among the earlier entries of its expert and the segment's count per expert;
//             then the experts' offsets; then each entry's place.
//  * products over the sorted rows: a tile of 64 rows belongs to one expert and reads that expert's matrix; the grid has
//             as many row tiles as the worst case needs (entries / 64 + experts) and the others leave at once.  Each output
//             is summed by one thread in k order, so a row's result does not depend on where the sort put it.
//  * combine: residual += sum over the choices (in their order) of weight x expert output, plus the shared expert's
//             output times its gate.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int SEG = 1024;

template <typename T, typename TW>
__global__ void __launch_bounds__(128)
route_kernel(int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ sgate, const T* __restrict__ h, long ldh,
             const TW* __restrict__ w_router, const TW* __restrict__ w_sg, int n_tokens, int width, int experts, int top) {
  extern __shared__ float sm[];            // [4 warps][experts] logits
  gi::pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n_tokens) return;
  float* lg = sm + (size_t)warp * experts;
  const T* hr = h + (size_t)t * ldh;
  for (int e = 0; e < experts; ++e) {
    const TW* wr = w_router + (size_t)e * width;
    float acc = 0.f;
    for (int i = lane; i < width; i += 32) acc = fmaf(gi::ldf(hr + i), gi::ldf(wr + i), acc);
    acc = gi::warp_sum(acc);
    if (lane == 0) lg[e] = acc;
  }
  if (w_sg != nullptr) {
    float acc = 0.f;
    for (int i = lane; i < width; i += 32) acc = fmaf(gi::ldf(hr + i), gi::ldf(w_sg + i), acc);
    acc = gi::warp_sum(acc);
    if (lane == 0) sgate[t] = 1.0f / (1.0f + expf(-acc));
  }
  __syncwarp();
  float first = 0.f, sum = 0.f, mine = 0.f;      // lane k keeps the k-th chosen logit (top <= 32)
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = lg[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = k < experts ? k : 0;      // every logit a NaN: any expert, never an index outside
    if (k == 0) first = best;
    const float ex = expf(best - first);
    sum += ex;
    if (lane == k) mine = ex;
    if (lane == 0) {
      ids[(size_t)t * top + k] = at;
      if (at < experts) lg[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane < top) wts[(size_t)t * top + lane] = mine / sum;
}

// ---- plan ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SEG)
rank_kernel(int* __restrict__ local_rank, int* __restrict__ seg_count, const int* __restrict__ ids, int entries, int experts) {
  extern __shared__ int smi[];             // [SEG] ids, [experts] histogram
  int* sid = smi;
  int* hist = smi + SEG;
  gi::pdl_prologue();
  const int seg = blockIdx.x, i = seg * SEG + threadIdx.x;
  const int id = i < entries ? ids[i] : -1;
  sid[threadIdx.x] = id;
  for (int e = threadIdx.x; e < experts; e += SEG) hist[e] = 0;
  __syncthreads();
  if (id >= 0) {
    int r = 0;
    for (int j = 0; j < (int)threadIdx.x; ++j) r += sid[j] == id;
    local_rank[i] = r;
    atomicAdd(&hist[id], 1);                // integer counts: the same whatever the order
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += SEG) seg_count[(size_t)seg * experts + e] = hist[e];
}

__global__ void __launch_bounds__(1024)
offsets_kernel(int* __restrict__ offsets, int* __restrict__ seg_count, int n_seg, int experts) {
  extern __shared__ int smi[];             // [experts] totals
  gi::pdl_prologue();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int run = 0;
    for (int s = 0; s < n_seg; ++s) {
      const int c = seg_count[(size_t)s * experts + e];
      seg_count[(size_t)s * experts + e] = run;     // becomes: entries of this expert in earlier segments
      run += c;
    }
    smi[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      run += smi[e];
    }
    offsets[experts] = run;
  }
}

__global__ void __launch_bounds__(SEG)
place_kernel(int* __restrict__ perm, int* __restrict__ inv, const int* __restrict__ offsets, const int* __restrict__ seg_base,
             const int* __restrict__ local_rank, const int* __restrict__ ids, int entries, int experts) {
  gi::pdl_prologue();
  const int seg = blockIdx.x, i = seg * SEG + threadIdx.x;
  if (i >= entries) return;
  const int id = ids[i];
  const int pos = offsets[id] + seg_base[(size_t)seg * experts + id] + local_rank[i];
  perm[pos] = i;
  inv[i] = pos;
}

// ---- products ----------------------------------------------------------------------------------------------------
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// Which expert and which rows row tile `ty` holds: experts in order, each with ceil(count / BM) tiles.
__device__ __forceinline__ bool tile_rows(const int* __restrict__ offsets, int experts, int ty, int* e_out, int* r0, int* r1) {
  int tiles = 0;
  for (int e = 0; e < experts; ++e) {
    const int lo = offsets[e], hi = offsets[e + 1];
    const int n = (hi - lo + BM - 1) / BM;
    if (ty < tiles + n) {
      *e_out = e;
      *r0 = lo + (ty - tiles) * BM;
      *r1 = min(hi, *r0 + BM);
      return true;
    }
    tiles += n;
  }
  return false;
}

// DUAL: two accumulators (gate rows n, up rows f + n of the expert's matrix), out = silu(gate) * up in the rows' type.
// else: out (float) = a W^T.
template <typename TA, typename TW, bool DUAL>
__global__ void __launch_bounds__(256)
expert_gemm_kernel(void* __restrict__ out_, const TA* __restrict__ A, long lda, const TW* __restrict__ W, long w_stride,
                   const int* __restrict__ offsets, const int* __restrict__ perm, int top, int experts, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[DUAL ? BK : 1][BN + 4];
  __shared__ int src[BM];
  gi::pdl_prologue();
  int e, r0, r1;
  if (!tile_rows(offsets, experts, blockIdx.y, &e, &r0, &r1)) return;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * BN;
  const TW* We = W + (size_t)e * w_stride;
  if (tid < BM) src[tid] = (r0 + tid < r1) ? (perm != nullptr ? perm[r0 + tid] / top : r0 + tid) : -1;
  __syncthreads();
  const int tx = tid % 16, ty = tid / 16;
  float acc[TM][TN], acu[DUAL ? TM : 1][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      acc[i][j] = 0.f;
      if (DUAL) acu[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int idx = tid + q * 256;
      const int r = idx / BK, kk = idx % BK, k = k0 + kk;
      float a = 0.f, w = 0.f, u = 0.f;
      if (k < K) {
        if (src[r] >= 0) a = gi::ldf(A + (size_t)src[r] * lda + k);
        if (n0 + r < N) {
          w = gi::ldf(We + (size_t)(n0 + r) * K + k);
          if (DUAL) u = gi::ldf(We + (size_t)(N + n0 + r) * K + k);
        }
      }
      As[kk][r] = a;
      Ws[kk][r] = w;
      if (DUAL) Us[kk][r] = u;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN], u[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        w[j] = Ws[kk][tx * TN + j];
        if (DUAL) u[j] = Us[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
          if (DUAL) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = r0 + ty * TM + i;
    if (r >= r1) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      if (DUAL) {
        const float g = acc[i][j];
        gi::stf((TA*)out_ + (size_t)r * N + n, g / (1.0f + expf(-g)) * acu[i][j]);
      } else {
        ((float*)out_)[(size_t)r * N + n] = acc[i][j];
      }
    }
  }
}

__global__ void __launch_bounds__(256)
combine_kernel(float* __restrict__ residual, const float* __restrict__ down, const int* __restrict__ inv,
               const float* __restrict__ wts, const float* __restrict__ shared, const float* __restrict__ sgate, int width,
               int top) {
  gi::pdl_prologue();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(wts[(size_t)t * top + k], down[(size_t)inv[(size_t)t * top + k] * width + i], acc);
    if (shared != nullptr) acc = fmaf(sgate[t], shared[(size_t)t * width + i], acc);
    residual[(size_t)t * width + i] += acc;
  }
}

}  // namespace

extern "C" int gi_moe_route(int* ids, float* wts, float* sgate, const void* h, int dtype, long ldh, const void* w_router,
                            const void* w_sg, int w_dtype, int n_tokens, int width, int experts, int top, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (experts < 1 || top < 1 || top > experts || top > 32 || experts > 8192)
    return gi::fail(GI_ERR_UNSUPPORTED, "router: %d of %d experts (at most 32 of 8192)", top, experts);
  if (w_sg != nullptr && sgate == nullptr) return gi::fail(GI_ERR_ARG, "router: a shared gate needs somewhere to go");
  const size_t smem = 4 * (size_t)experts * sizeof(float);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW, {
      auto kern = route_kernel<T, TW>;
      if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess)
        e = gi::launch(kern, dim3((n_tokens + 3) / 4), dim3(128), smem, (cudaStream_t)stream, ids, wts, sgate, (const T*)h, ldh,
                       (const TW*)w_router, (const TW*)w_sg, n_tokens, width, experts, top);
  }));
  return gi::check(e, "router");
}

extern "C" int gi_moe_plan(int* offsets, int* perm, int* inv, int* scratch, const int* ids, int entries, int experts,
                           void* stream) {
  if (entries <= 0) return GI_OK;
  if (experts < 1 || experts > 8192) return gi::fail(GI_ERR_UNSUPPORTED, "router plan: %d experts (at most 8192)", experts);
  const int n_seg = (entries + SEG - 1) / SEG;
  int* seg_count = scratch;                          // [n_seg][experts]
  int* local_rank = scratch + (size_t)n_seg * experts;   // [entries]
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = gi::launch(rank_kernel, dim3(n_seg), dim3(SEG), (SEG + (size_t)experts) * sizeof(int), s, local_rank, seg_count,
                             ids, entries, experts);
  if (e == cudaSuccess)
    e = gi::launch(offsets_kernel, dim3(1), dim3(experts < 1024 ? ((experts + 31) / 32) * 32 : 1024), (size_t)experts * sizeof(int),
                   s, offsets, seg_count, n_seg, experts);
  if (e == cudaSuccess)
    e = gi::launch(place_kernel, dim3(n_seg), dim3(SEG), 0, s, perm, inv, (const int*)offsets, (const int*)seg_count,
                   (const int*)local_rank, ids, entries, experts);
  return gi::check(e, "router plan");
}

extern "C" int gi_moe_gemm_gate_up(void* out, int dtype, const void* a, long lda, const void* w, int w_dtype, long w_stride,
                                   const int* offsets, const int* perm, int entries, int top, int experts, int f, int k,
                                   void* stream) {
  if (entries <= 0) return GI_OK;
  if (f <= 0 || k <= 0 || top < 1) return gi::fail(GI_ERR_ARG, "expert product: bad sizes");
  const long tiles = (entries + BM - 1) / BM + experts;
  if (tiles > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "expert product: %d rows are more than one launch takes", entries);
  dim3 grid((f + BN - 1) / BN, (unsigned)tiles);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, TA, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(expert_gemm_kernel<TA, TW, true>, grid, dim3(256), 0, (cudaStream_t)stream, out, (const TA*)a, lda,
                     (const TW*)w, w_stride, offsets, perm, top, experts, f, k)));
  return gi::check(e, "expert product (gate, up)");
}

extern "C" int gi_moe_gemm_down(float* out, const void* a, int dtype, long lda, const void* w, int w_dtype, long w_stride,
                                const int* offsets, int entries, int experts, int n, int k, void* stream) {
  if (entries <= 0) return GI_OK;
  if (n <= 0 || k <= 0) return gi::fail(GI_ERR_ARG, "expert product: bad sizes");
  const long tiles = (entries + BM - 1) / BM + experts;
  if (tiles > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "expert product: %d rows are more than one launch takes", entries);
  dim3 grid((n + BN - 1) / BN, (unsigned)tiles);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, TA, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(expert_gemm_kernel<TA, TW, false>, grid, dim3(256), 0, (cudaStream_t)stream, (void*)out, (const TA*)a, lda,
                     (const TW*)w, w_stride, offsets, (const int*)nullptr, 1, experts, n, k)));
  return gi::check(e, "expert product (down)");
}

extern "C" int gi_moe_combine(float* residual, const float* down, const int* inv, const float* wts, const float* shared,
                              const float* sgate, int n_tokens, int width, int top, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (shared != nullptr && sgate == nullptr) return gi::fail(GI_ERR_ARG, "expert combine: a shared output needs its gate");
  return gi::check(gi::launch(combine_kernel, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, residual, down, inv, wts, shared,
                              sgate, width, top), "expert combine");
}
