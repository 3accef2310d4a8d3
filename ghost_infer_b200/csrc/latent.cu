// Row kernels and small products for layers whose attention keeps one low-rank latent per token instead of keys and
// values per head, and for feed-forwards with biases and a squared relu.
//
//  * layernorm:        y = (x - mean) / sqrt(var + eps) * w, statistics in 32-bit, one block per row.
//  * bias_act:         out = act(in + bias) over rows, and (optionally, in the same launch) residual rows += a bias.
//  * latent_prepare:   one token's row [query latent | key/value latent | shared rotary key part] of the down product:
//                      the query latent is RMS-normed for the next product; the key/value latent is RMS-normed and,
//                      with the rotated key part behind it, written to the token's place in the paged cache.
//  * latent_query_rot: the rotary part of every head's query, rotated, into the rows the attention reads
//                      ([heads][latent | rotary part]); the latent part of those rows comes from bmm_heads.
//  * bmm_heads:        out[t, h, :] = W_h a[t, h, :], one small matrix per head (the keys' up-projection folded onto the
//                      queries, the values' up-projection applied to the attention's output).
#include <math.h>

#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

// ---- layer norm --------------------------------------------------------------------------------------------------
// The order of every sum follows from the width alone (256 threads, a fixed tree), so a row gives the same bits in any step.
template <typename TO, typename TW>
__global__ void __launch_bounds__(256)
layernorm_kernel(TO* __restrict__ out, const float* x, const TW* __restrict__ w, const int* rows, int d, float eps) {
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const int r = blockIdx.x;
  const int m = rows ? rows[r] : r;
  const float* xr = x + (size_t)m * d;
  TO* o = out + (size_t)r * d;
  constexpr int PER = 8;
  const bool in_regs = d <= PER * 256;
  float v[PER];
  float s = 0.f;
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * 256;
      v[j] = i < d ? xr[i] : 0.f;
      s += v[j];
    }
  } else {
    for (int i = threadIdx.x; i < d; i += 256) s += xr[i];
  }
  const float mean = gi::block_sum(s, scratch) / (float)d;
  float q = 0.f;
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * 256;
      const float dv = i < d ? v[j] - mean : 0.f;
      q = fmaf(dv, dv, q);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += 256) {
      const float dv = xr[i] - mean;
      q = fmaf(dv, dv, q);
    }
  }
  const float rstd = 1.0f / sqrtf(gi::block_sum(q, scratch) / (float)d + eps);
  if (in_regs) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int i = threadIdx.x + j * 256;
      if (i < d) gi::stf(o + i, (v[j] - mean) * rstd * gi::ldf(w + i));
    }
  } else {
    for (int i = threadIdx.x; i < d; i += 256) gi::stf(o + i, (xr[i] - mean) * rstd * gi::ldf(w + i));
  }
}

// The same with a row in registers as float4 (widths that are multiples of 4, up to 4096, rows on 16-byte boundaries), and,
// SETTLE, first adding the partial sums a deferred product left for the rows it reads (written back to x unless `rows`
// selects: then x is left as it is and must not be read again).
__device__ __forceinline__ float4 pending_sum4(const gi_settle_t& st, int m, int f) {
  const gi_settle_span sp = gi_span_of(st, f);
  if (sp.c_first == sp.c_last) return make_float4(0.f, 0.f, 0.f, 0.f);     // one block had the whole tile and added it itself
  return gi_sum_pieces4(st, sp, m, f);
}

template <typename TO, typename TW, bool SETTLE>
__global__ void __launch_bounds__(256)
layernorm_vec_kernel(TO* __restrict__ out, float* x, const TW* __restrict__ w, const int* rows, int d, float eps, gi_settle_t st) {
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const int r = blockIdx.x;
  const int m = rows ? rows[r] : r;
  float4* xr = reinterpret_cast<float4*>(x + (size_t)m * d);
  TO* o = out + (size_t)r * d;
  const int n4 = d / 4;
  float4 v[4];
  float s = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + j * 256;
    v[j] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    if (SETTLE && i < n4) {
      const float4 p = pending_sum4(st, m, 4 * i);
      v[j].x += p.x;
      v[j].y += p.y;
      v[j].z += p.z;
      v[j].w += p.w;
      if (rows == nullptr) xr[i] = v[j];
    }
    s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
  }
  const float mean = gi::block_sum(s, scratch) / (float)d;
  float q = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < n4) {
      const float a = v[j].x - mean, b = v[j].y - mean, c = v[j].z - mean, e = v[j].w - mean;
      q = fmaf(a, a, q);
      q = fmaf(b, b, q);
      q = fmaf(c, c, q);
      q = fmaf(e, e, q);
    }
  }
  const float rstd = 1.0f / sqrtf(gi::block_sum(q, scratch) / (float)d + eps);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int i = threadIdx.x + j * 256;
    if (i < n4) {
      gi::stf(o + 4 * i, (v[j].x - mean) * rstd * gi::ldf(w + 4 * i));
      gi::stf(o + 4 * i + 1, (v[j].y - mean) * rstd * gi::ldf(w + 4 * i + 1));
      gi::stf(o + 4 * i + 2, (v[j].z - mean) * rstd * gi::ldf(w + 4 * i + 2));
      gi::stf(o + 4 * i + 3, (v[j].w - mean) * rstd * gi::ldf(w + 4 * i + 3));
    }
  }
}

// ---- bias and activation -------------------------------------------------------------------------------------------
// act 0: none; 1: relu(z)^2.
template <typename T, typename TW>
__global__ void bias_act_kernel(T* __restrict__ out, const T* in, long ld_in, const TW* __restrict__ bias, int f, size_t total_act,
                                int act, float* residual, const TW* __restrict__ res_bias, int d, size_t total) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  if (i < total_act) {
    const size_t m = i / f, c = i % f;
    float z = gi::ldf(in + m * ld_in + c);
    if (bias != nullptr) z += gi::ldf(bias + c);
    if (act == 1) {
      z = fmaxf(z, 0.f);
      z *= z;
    }
    gi::stf(out + i, z);
  } else {
    const size_t k = i - total_act;
    residual[k] += gi::ldf(res_bias + k % d);
  }
}

// ---- the latent's row --------------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(T* __restrict__ cq, const T* in, long ld, const TW* __restrict__ wq, const TW* __restrict__ wc, float eps,
                      const float2* table, int half, const int* positions, const int* slots, const int* block_table,
                      int max_pages, T* kcache, int rq, int r, int dr, int write_cache) {
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const int t = blockIdx.x;
  const T* row = in + (size_t)t * ld;
  // the queries' latent: x / sqrt(mean(x^2) + eps) * w
  if (rq > 0) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < rq; i += 128) {
      const float v = gi::ldf(row + i);
      ss = fmaf(v, v, ss);
    }
    const float rs = 1.0f / sqrtf(gi::block_sum(ss, scratch) / (float)rq + eps);
    for (int i = threadIdx.x; i < rq; i += 128) gi::stf(cq + (size_t)t * rq + i, gi::ldf(row + i) * rs * gi::ldf(wq + i));
  }
  if (!write_cache) return;
  const int slot = slots[t];
  const int pos = max(positions[t], 0);
  const int page = slot >= 0 ? block_table[(size_t)slot * max_pages + pos / PAGE_TOKENS] : 0;
  T* dst = kcache + ((size_t)page * PAGE_TOKENS + pos % PAGE_TOKENS) * (size_t)(r + dr);
  const T* lat = row + rq;
  float ss = 0.f;
  for (int i = threadIdx.x; i < r; i += 128) {
    const float v = gi::ldf(lat + i);
    ss = fmaf(v, v, ss);
  }
  const float rs = 1.0f / sqrtf(gi::block_sum(ss, scratch) / (float)r + eps);
  for (int i = threadIdx.x; i < r; i += 128) gi::stf(dst + i, gi::ldf(lat + i) * rs * gi::ldf(wc + i));
  // the key part all heads share: its first 2 * half numbers turn in neighbouring pairs, the rest pass
  const T* kr = lat + r;
  for (int i = threadIdx.x; i < half; i += 128) {
    float a, b;
    gi::rotate_pair(gi::ldf(kr + 2 * i), gi::ldf(kr + 2 * i + 1), table[(size_t)t * half + i], &a, &b);
    gi::stf(dst + r + 2 * i, a);
    gi::stf(dst + r + 2 * i + 1, b);
  }
  for (int i = 2 * half + threadIdx.x; i < dr; i += 128) dst[r + i] = kr[i];
}

// The same with 16-byte accesses and the row kept in registers: bfloat16, every part a multiple of 8 numbers wide, rows on
// 16-byte boundaries, at most 4096 numbers in the two latents together.  A thread holds up to two chunks of 8 numbers; both
// sums of squares go through the block at once.
template <typename TW>
__global__ void __launch_bounds__(256)
latent_prepare_vec_kernel(__nv_bfloat16* __restrict__ cq, const __nv_bfloat16* in, long ld, const TW* __restrict__ wq,
                          const TW* __restrict__ wc, float eps, const float2* table, int half, const int* positions,
                          const int* slots, const int* block_table, int max_pages, __nv_bfloat16* kcache, int rq, int r, int dr,
                          int write_cache) {
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const int t = blockIdx.x;
  const __nv_bfloat16* row = in + (size_t)t * ld;
  const int nq = rq / 8, nc = r / 8;               // chunks of the two latents
  float v[2][8];
  float ssq = 0.f, ssc = 0.f;
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int ci = threadIdx.x + j * 256;
    if (ci < nq + nc) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + ci * 8);
      const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[j][2 * i] = __uint_as_float(w4[i] << 16);
        v[j][2 * i + 1] = __uint_as_float(w4[i] & 0xffff0000u);
        ss = fmaf(v[j][2 * i], v[j][2 * i], ss);
        ss = fmaf(v[j][2 * i + 1], v[j][2 * i + 1], ss);
      }
      if (ci < nq) ssq += ss; else ssc += ss;
    }
  }
  const float rsq = rq > 0 ? 1.0f / sqrtf(gi::block_sum(ssq, scratch) / (float)rq + eps) : 0.f;
  const float rsc = 1.0f / sqrtf(gi::block_sum(ssc, scratch) / (float)r + eps);
  __nv_bfloat16* dst = nullptr;
  if (write_cache) {
    const int slot = slots[t];
    const int pos = max(positions[t], 0);
    const int page = slot >= 0 ? block_table[(size_t)slot * max_pages + pos / PAGE_TOKENS] : 0;
    dst = kcache + ((size_t)page * PAGE_TOKENS + pos % PAGE_TOKENS) * (size_t)(r + dr);
  }
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int ci = threadIdx.x + j * 256;
    if (ci >= nq + nc) continue;
    const bool is_q = ci < nq;
    if (!is_q && !write_cache) continue;
    const TW* w = is_q ? wq + ci * 8 : wc + (ci - nq) * 8;
    const float rs = is_q ? rsq : rsc;
    uint32_t p[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) p[i] = gi::pack_bf16(v[j][2 * i] * rs * gi::ldf(w + 2 * i), v[j][2 * i + 1] * rs * gi::ldf(w + 2 * i + 1));
    __nv_bfloat16* o = is_q ? cq + (size_t)t * rq + ci * 8 : dst + (ci - nq) * 8;
    *reinterpret_cast<uint4*>(o) = make_uint4(p[0], p[1], p[2], p[3]);
  }
  if (!write_cache) return;
  const __nv_bfloat16* kr = row + rq + r;
  for (int i = threadIdx.x; i < half; i += 256) {
    float a, b;
    gi::rotate_pair(gi::ldf(kr + 2 * i), gi::ldf(kr + 2 * i + 1), table[(size_t)t * half + i], &a, &b);
    gi::stf(dst + r + 2 * i, a);
    gi::stf(dst + r + 2 * i + 1, b);
  }
  for (int i = 2 * half + threadIdx.x; i < dr; i += 256) dst[r + i] = kr[i];
}

template <typename T>
__global__ void __launch_bounds__(256)
latent_query_rot_kernel(T* qa, long ldqa, const T* q, long ldq, const float2* table, int half, int n_heads, int dn, int dr, int r) {
  gi::pdl_prologue();
  const int t = blockIdx.x;
  const int per = dr - half;                       // work items of a head: `half` pairs, then dr - 2 half numbers that pass
  for (int idx = threadIdx.x; idx < n_heads * per; idx += 256) {
    const int h = idx / per, i = idx % per;
    const T* src = q + (size_t)t * ldq + (size_t)h * (dn + dr) + dn;
    T* dst = qa + (size_t)t * ldqa + (size_t)h * (r + dr) + r;
    if (i < half) {
      float a, b;
      gi::rotate_pair(gi::ldf(src + 2 * i), gi::ldf(src + 2 * i + 1), table[(size_t)t * half + i], &a, &b);
      gi::stf(dst + 2 * i, a);
      gi::stf(dst + 2 * i + 1, b);
    } else {
      dst[half + i] = src[half + i];
    }
  }
}

// ---- one small product per head, CUDA cores ------------------------------------------------------------------------
// out[t, h * ohs + n] = sum_k a[t, h * ahs + k] * W[h * whs + n * ldw + k * kstride]; every output is summed by one thread
// in k order, so a row's result does not depend on the step's other rows.
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
bmm_heads_kernel(TO* __restrict__ out, long ldo, long ohs, const TA* A, long lda, long ahs, const TW* __restrict__ W, long whs,
                 long ldw, long kstride, int M, int N, int K) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  gi::pdl_prologue();
  const int h = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const TA* Ah = A + (size_t)h * ahs;
  const TW* Wh = W + (size_t)h * whs;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int idx = tid + q * 256;
      const int rr = idx / BK, kk = idx % BK, k = k0 + kk;
      float a = 0.f, w = 0.f;
      if (k < K) {
        if (m0 + rr < M) a = gi::ldf(Ah + (size_t)(m0 + rr) * lda + k);
        if (n0 + rr < N) w = gi::ldf(Wh + (size_t)(n0 + rr) * ldw + (size_t)k * kstride);
      }
      As[kk][rr] = a;
      Ws[kk][rr] = w;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int m = m0 + ty * TM + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) gi::stf(out + (size_t)m * ldo + (size_t)h * ohs + n, acc[i][j]);
    }
  }
}

// ---- the same on tensor cores: bfloat16 in and out, W_h stored [N][K] row-major (kstride 1) -------------------------------
// A block takes 64 rows x 64 columns of one head: four warps of 16 rows each, `mma.sync m16n8k16` with 32-bit sums; the
// operands of a 32-wide slice of K go through shared memory (rows padded to 40 values, so that the fragments' loads
// meet no bank twice).  Edges are filled with zeros and not stored.  VEC: every row of both operands starts on a 16-byte
// boundary and K is a multiple of 8, so the slices arrive by `cp.async`, 16 bytes a copy, the next slice under way while
// this one is multiplied; else element by element, one slice at a time.
constexpr int TK = 32, TLD = TK + 8;

template <bool VEC>
__global__ void __launch_bounds__(128)
bmm_heads_mma_kernel(__nv_bfloat16* __restrict__ out, long ldo, long ohs, const __nv_bfloat16* A, long lda, long ahs,
                     const __nv_bfloat16* __restrict__ W, long whs, long ldw, int M, int N, int K) {
  __shared__ __align__(16) __nv_bfloat16 As[2][64 * TLD];
  __shared__ __align__(16) __nv_bfloat16 Ws[2][64 * TLD];
  gi::pdl_prologue();
  const int h = blockIdx.z, m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const __nv_bfloat16* Ah = A + (size_t)h * ahs;
  const __nv_bfloat16* Wh = W + (size_t)h * whs;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, c = lane & 3;
  float acc[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[j][i] = 0.f;
  const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
  const int n_slices = (K + TK - 1) / TK;

  auto fill = [&](int slice, int stage) {
    const int k0 = slice * TK;
    if (VEC) {
      // 64 rows x 4 chunks of 8 values per operand: two chunks of each per thread
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int idx = tid + i * 128;
        const int rr = idx >> 2, kk = (idx & 3) * 8, k = k0 + kk;
        const int oka = (m0 + rr < M && k < K) ? 16 : 0, okw = (n0 + rr < N && k < K) ? 16 : 0;
        gi::cp_async_16(gi::smem_u32(&As[stage][rr * TLD + kk]), Ah + (oka ? (size_t)(m0 + rr) * lda + k : 0), oka);
        gi::cp_async_16(gi::smem_u32(&Ws[stage][rr * TLD + kk]), Wh + (okw ? (size_t)(n0 + rr) * ldw + k : 0), okw);
      }
    } else {
      for (int idx = tid; idx < 64 * TK; idx += 128) {
        const int rr = idx / TK, kk = idx % TK, k = k0 + kk;
        As[stage][rr * TLD + kk] = (m0 + rr < M && k < K) ? Ah[(size_t)(m0 + rr) * lda + k] : zero;
        Ws[stage][rr * TLD + kk] = (n0 + rr < N && k < K) ? Wh[(size_t)(n0 + rr) * ldw + k] : zero;
      }
    }
  };

  fill(0, 0);
  if (VEC) gi::cp_async_commit();
  for (int sl = 0; sl < n_slices; ++sl) {
    const int stage = VEC ? (sl & 1) : 0;
    if (VEC) {
      if (sl + 1 < n_slices) fill(sl + 1, stage ^ 1);
      gi::cp_async_commit();
      gi::cp_async_wait<1>();
    }
    __syncthreads();
#pragma unroll
    for (int ks = 0; ks < TK; ks += 16) {
      uint32_t a[4];
      const __nv_bfloat16* ar = &As[stage][(warp * 16 + g) * TLD + ks + 2 * c];
      a[0] = *reinterpret_cast<const uint32_t*>(ar);
      a[1] = *reinterpret_cast<const uint32_t*>(ar + 8 * TLD);
      a[2] = *reinterpret_cast<const uint32_t*>(ar + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(ar + 8 * TLD + 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const __nv_bfloat16* wr = &Ws[stage][(j * 8 + g) * TLD + ks + 2 * c];
        gi::mma_16816(acc[j], a, *reinterpret_cast<const uint32_t*>(wr), *reinterpret_cast<const uint32_t*>(wr + 8));
      }
    }
    __syncthreads();
    if (!VEC && sl + 1 < n_slices) fill(sl + 1, 0);
  }
  const int r_lo = m0 + warp * 16 + g, r_hi = r_lo + 8;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int n = n0 + j * 8 + 2 * c;
    if (n < N) {
      if (r_lo < M) out[(size_t)r_lo * ldo + (size_t)h * ohs + n] = __float2bfloat16_rn(acc[j][0]);
      if (r_hi < M) out[(size_t)r_hi * ldo + (size_t)h * ohs + n] = __float2bfloat16_rn(acc[j][2]);
    }
    if (n + 1 < N) {
      if (r_lo < M) out[(size_t)r_lo * ldo + (size_t)h * ohs + n + 1] = __float2bfloat16_rn(acc[j][1]);
      if (r_hi < M) out[(size_t)r_hi * ldo + (size_t)h * ohs + n + 1] = __float2bfloat16_rn(acc[j][3]);
    }
  }
}

// ---- the same for a step of few rows (one-token steps): bound by the bytes of the heads' matrices ------------------------
// grid (column tiles of 16, heads); a block stages up to 8 rows' numbers for its head in shared memory and streams 16 rows of
// the head's matrix past them, 16 bytes per lane per load, four columns in flight; a warp takes 4 columns, its lanes cut K
// between them and their sums meet in a fixed order.  bfloat16, K a multiple of 8, rows on 16-byte boundaries.
constexpr int GV_ROWS = 8, GV_COLS = 16;      // a warp takes 4 columns

__global__ void __launch_bounds__(128)
bmm_heads_gemv_kernel(__nv_bfloat16* __restrict__ out, long ldo, long ohs, const __nv_bfloat16* A, long lda, long ahs,
                      const __nv_bfloat16* __restrict__ W, long whs, long ldw, int M, int N, int K) {
  extern __shared__ __align__(16) unsigned char gv_smem[];
  __nv_bfloat16* As = reinterpret_cast<__nv_bfloat16*>(gv_smem);      // [GV_ROWS][K]
  gi::pdl_prologue();
  const int h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __nv_bfloat16* Ah = A + (size_t)h * ahs;
  const __nv_bfloat16* Wh = W + (size_t)h * whs;
  const int n_base = blockIdx.x * GV_COLS + warp * 4;
  for (int r0 = 0; r0 < M; r0 += GV_ROWS) {
    const int rows = min(GV_ROWS, M - r0);
    __syncthreads();
    for (int idx = tid; idx < rows * (K / 8); idx += 128) {
      const int r = idx / (K / 8), ch = idx % (K / 8);
      *reinterpret_cast<uint4*>(As + (size_t)r * K + ch * 8) = *reinterpret_cast<const uint4*>(Ah + (size_t)(r0 + r) * lda + ch * 8);
    }
    __syncthreads();
    for (int j0 = 0; j0 < 4; j0 += 4) {
      if (n_base + j0 >= N) break;                      // the same for the whole warp
      const __nv_bfloat16* wp[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) wp[jj] = Wh + (size_t)min(n_base + j0 + jj, N - 1) * ldw;     // past the end: repeated, not stored
      float acc[4][GV_ROWS];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) acc[jj][r] = 0.f;
      for (int k = lane * 8; k < K; k += 256) {
        uint4 wv[4];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) wv[jj] = *reinterpret_cast<const uint4*>(wp[jj] + k);
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) {
          if (r < rows) {
            const uint4 av = *reinterpret_cast<const uint4*>(As + (size_t)r * K + k);
            const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const uint32_t ww[4] = {wv[jj].x, wv[jj].y, wv[jj].z, wv[jj].w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                acc[jj][r] = fmaf(__uint_as_float(aw[i] << 16), __uint_as_float(ww[i] << 16), acc[jj][r]);
                acc[jj][r] = fmaf(__uint_as_float(aw[i] & 0xffff0000u), __uint_as_float(ww[i] & 0xffff0000u), acc[jj][r]);
              }
            }
          }
        }
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int n = n_base + j0 + jj;
#pragma unroll
        for (int r = 0; r < GV_ROWS; ++r) {
          if (r >= rows) break;
          const float v = gi::warp_sum(acc[jj][r]);
          if (lane == 0 && n < N) out[(size_t)(r0 + r) * ldo + (size_t)h * ohs + n] = __float2bfloat16_rn(v);
        }
      }
    }
  }
}

}  // namespace

extern "C" int gi_layernorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype, const int* rows, int n_rows,
                            int d, float eps, void* stream) {
  gi_settle_t none = {nullptr, nullptr, nullptr, nullptr, 0};
  return gi_layernorm_settle(out, out_dtype, const_cast<float*>(x), w, w_dtype, rows, n_rows, d, eps, none, stream);
}

extern "C" int gi_layernorm_settle(void* out, int out_dtype, float* x, const void* w, int w_dtype, const int* rows, int n_rows,
                                   int d, float eps, gi_settle_t settle, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (d <= 0) return gi::fail(GI_ERR_ARG, "layernorm: bad width %d", d);
  cudaError_t e = cudaSuccess;
  const bool vec = d % 4 == 0 && d <= 4096 && !((uintptr_t)x & 15);
  if (settle.partials != nullptr && !vec)
    return gi::fail(GI_ERR_UNSUPPORTED, "layernorm: settling partial sums needs rows of a multiple of 4 and at most 4096 values");
  if (vec) {
    if (settle.partials != nullptr)
      GI_DISPATCH_DTYPE(out_dtype, TO, GI_DISPATCH_DTYPE(w_dtype, TW,
          e = gi::launch(layernorm_vec_kernel<TO, TW, true>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, (TO*)out, x, (const TW*)w, rows, d, eps, settle)));
    else
      GI_DISPATCH_DTYPE(out_dtype, TO, GI_DISPATCH_DTYPE(w_dtype, TW,
          e = gi::launch(layernorm_vec_kernel<TO, TW, false>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, (TO*)out, x, (const TW*)w, rows, d, eps, settle)));
    return gi::check(e, "layernorm");
  }
  GI_DISPATCH_DTYPE(out_dtype, TO, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(layernorm_kernel<TO, TW>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, (TO*)out, x, (const TW*)w, rows, d, eps)));
  return gi::check(e, "layernorm");
}

extern "C" int gi_bias_act(void* out, const void* in, int dtype, long ld_in, const void* bias, int w_dtype, int n_rows, int f,
                           int act, float* residual, const void* res_bias, int d, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (f < 0 || (f == 0 && residual == nullptr) || (act != 0 && act != 1))
    return gi::fail(GI_ERR_ARG, "bias_act: bad width %d or activation %d", f, act);
  if ((residual != nullptr) != (res_bias != nullptr) || (residual != nullptr && d <= 0))
    return gi::fail(GI_ERR_ARG, "bias_act: a bias for the residual rows needs both the rows and the bias");
  const size_t total_act = (size_t)n_rows * f;
  const size_t total = total_act + (residual != nullptr ? (size_t)n_rows * d : 0);
  const unsigned blocks = (unsigned)((total + 255) / 256);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(bias_act_kernel<T, TW>, dim3(blocks), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)in, ld_in,
                     (const TW*)bias, f, total_act, act, residual, (const TW*)res_bias, d, total)));
  return gi::check(e, "bias_act");
}

extern "C" int gi_latent_prepare(void* cq, const void* in, int dtype, long ld, const void* wq, const void* wc, int w_dtype,
                                 float eps, const float* table, int rot, const int* positions, const int* slots,
                                 const int* block_table, int max_pages, void* kcache, int n_tokens, int rq, int r, int dr,
                                 int write_cache, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (rq < 0 || r <= 0 || dr < 0 || rot < 0 || rot % 2 != 0 || rot > dr)
    return gi::fail(GI_ERR_ARG, "latent rows: bad sizes (query latent %d, latent %d, rotary part %d of which %d turn)", rq, r, dr, rot);
  if (rot > 0 && table == nullptr) return gi::fail(GI_ERR_ARG, "latent rows: no table of angles");
  if (write_cache && (!kcache || !block_table || !slots || !positions)) return gi::fail(GI_ERR_ARG, "latent rows: cache write without a cache");
  cudaError_t e = cudaSuccess;
  if (dtype == GI_BF16 && rq % 8 == 0 && r % 8 == 0 && dr % 8 == 0 && ld % 8 == 0 && rq + r <= 4096 &&
      !(((uintptr_t)in | (uintptr_t)cq | (uintptr_t)kcache) & 15) && !(((uintptr_t)wq | (uintptr_t)wc) & 15)) {
    GI_DISPATCH_DTYPE(w_dtype, TW,
        e = gi::launch(latent_prepare_vec_kernel<TW>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, (__nv_bfloat16*)cq,
                       (const __nv_bfloat16*)in, ld, (const TW*)wq, (const TW*)wc, eps, (const float2*)table, rot / 2, positions, slots,
                       block_table, max_pages, (__nv_bfloat16*)kcache, rq, r, dr, write_cache));
    return gi::check(e, "latent rows");
  }
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(latent_prepare_kernel<T, TW>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (T*)cq, (const T*)in, ld,
                     (const TW*)wq, (const TW*)wc, eps, (const float2*)table, rot / 2, positions, slots, block_table, max_pages,
                     (T*)kcache, rq, r, dr, write_cache)));
  return gi::check(e, "latent rows");
}

extern "C" int gi_latent_query_rot(void* qa, long ldqa, const void* q, long ldq, int dtype, const float* table, int rot,
                                   int n_tokens, int n_heads, int dn, int dr, int r, void* stream) {
  if (n_tokens <= 0 || dr <= 0) return GI_OK;
  if (rot < 0 || rot % 2 != 0 || rot > dr || n_heads <= 0 || n_heads > 65535)
    return gi::fail(GI_ERR_ARG, "latent queries: bad sizes (%d heads, rotary part %d of which %d turn)", n_heads, dr, rot);
  if (rot > 0 && table == nullptr) return gi::fail(GI_ERR_ARG, "latent queries: no table of angles");
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(latent_query_rot_kernel<T>, dim3(n_tokens), dim3(256), 0, (cudaStream_t)stream, (T*)qa, ldqa,
                     (const T*)q, ldq, (const float2*)table, rot / 2, n_heads, dn, dr, r));
  return gi::check(e, "latent queries");
}

extern "C" int gi_bmm_heads(void* out, long ldo, long ohs, const void* a, long lda, long ahs, int dtype, const void* w, int w_dtype,
                            long whs, long ldw, long kstride, int M, int N, int K, int heads, int tensor_cores, void* stream) {
  if (M <= 0 || heads <= 0) return GI_OK;
  if (N <= 0 || K <= 0) return gi::fail(GI_ERR_ARG, "per-head product: bad sizes N=%d K=%d", N, K);
  const long my = (M + 63) / 64;
  if (heads > 65535 || my > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "per-head product: more than 65535 heads or row tiles");
  dim3 grid((N + 63) / 64, (unsigned)my, heads);
  cudaError_t e = cudaSuccess;
  if (tensor_cores && dtype == GI_BF16 && w_dtype == GI_BF16 && kstride == 1 && lda % 2 == 0 && ahs % 2 == 0 && ldw % 2 == 0 &&
      whs % 2 == 0 && !(((uintptr_t)a | (uintptr_t)w) & 3)) {
    const bool vec = K % 8 == 0 && lda % 8 == 0 && ahs % 8 == 0 && ldw % 8 == 0 && whs % 8 == 0 && !(((uintptr_t)a | (uintptr_t)w) & 15);
    if (vec && M <= 32 && (size_t)GV_ROWS * K * 2 <= 96 * 1024) {
      // few rows: the matrices are streamed once
      const size_t smem = (size_t)GV_ROWS * K * 2;
      static size_t configured[gi::MAX_DEVICES_SEEN] = {0};
      int dev = -1;
      if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= gi::MAX_DEVICES_SEEN) dev = -1;
      if (smem > 48 * 1024 && (dev < 0 || configured[dev] < smem)) {
        e = cudaFuncSetAttribute(bmm_heads_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "per-head product: %s", cudaGetErrorString(e));
        if (dev >= 0) configured[dev] = smem;
      }
      e = gi::launch(bmm_heads_gemv_kernel, dim3((N + GV_COLS - 1) / GV_COLS, heads), dim3(128), smem, (cudaStream_t)stream,
                     (__nv_bfloat16*)out, ldo, ohs, (const __nv_bfloat16*)a, lda, ahs, (const __nv_bfloat16*)w, whs, ldw, M, N, K);
      return gi::check(e, "per-head product (few rows)");
    }
    if (vec)
      e = gi::launch(bmm_heads_mma_kernel<true>, grid, dim3(128), 0, (cudaStream_t)stream, (__nv_bfloat16*)out, ldo, ohs,
                     (const __nv_bfloat16*)a, lda, ahs, (const __nv_bfloat16*)w, whs, ldw, M, N, K);
    else
      e = gi::launch(bmm_heads_mma_kernel<false>, grid, dim3(128), 0, (cudaStream_t)stream, (__nv_bfloat16*)out, ldo, ohs,
                     (const __nv_bfloat16*)a, lda, ahs, (const __nv_bfloat16*)w, whs, ldw, M, N, K);
    return gi::check(e, "per-head product");
  }
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(bmm_heads_kernel<T, TW, T>, grid, dim3(256), 0, (cudaStream_t)stream, (T*)out, ldo, ohs, (const T*)a, lda, ahs,
                     (const TW*)w, whs, ldw, kstride, M, N, K)));
  return gi::check(e, "per-head product");
}
