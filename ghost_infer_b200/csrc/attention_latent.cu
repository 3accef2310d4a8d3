// Causal attention of many heads over ONE shared row per position (a low-rank latent that is key and value at once), on
// tensor cores: bfloat16, `mma.sync m16n8k16`, 32-bit scores, softmax statistics and sums.
//
// The cache holds rows [latent (dv) | rotary key part] of dk numbers, pages of 64 positions.  A head's query row has the
// same layout; its score with a position is their product times `scale`, and the position's value is the row's first dv
// numbers.  Since every head reads the same rows, the rows of the tensor-core tile are (token, head) pairs: 64 of them a
// block in a prompt step (row i of a sequence's step is token i / heads, head i % heads; its causal limit is its token's
// position), the heads of one token in a one-token step.  A key tile (one page, 64 x dk) is fetched once by `cp.async`
// into a two-stage ring and serves the score product (all dk columns) and the output product (its first dv columns).
//
//  * rows mode (prompts; one-token steps with more than 16 heads): four warps of 16 rows each walk every tile.
//  * keys mode (one-token steps with at most 16 heads): the four warps share the 16 rows and take 16 keys of a tile
//    each; their running maxima, sums and outputs meet in shared memory at the end, in warp order.
//  In both, with values wider than 256, a second set of four warps repeats the scores and takes the values' upper half
//  (a thread cannot hold more than 16 x 256 / 32 sums).
//  One-token steps cut the context into slices (grid.y); slices are merged by gi_attn_combine.
// Sizes: dk and dv multiples of 8, dk <= 576, dv <= 512.  Queries' key columns and the tiles' are padded with zeros to a
// multiple of 16; rows in shared memory are 8 values longer than that, which keeps `ldmatrix` free of bank conflicts.
#include <math.h>

#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int BQ = 64, BKV = 64;
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

template <int NVT, int DSPLIT, bool KEYS>
__global__ void __launch_bounds__(128 * DSPLIT)
attn_latent_mma_kernel(__nv_bfloat16* __restrict__ out, long ldo, float* __restrict__ part_o, float* __restrict__ part_ml,
                       const __nv_bfloat16* q, long ldq, const __nv_bfloat16* kcache, const int* block_table, int max_pages,
                       const int* cu_seqlens, const int* seq_slots, const int* seq_pos0, const int* seq_lens, int n_heads,
                       float scale, int dk, int dv, int hd, int n_splits, int own_tiles) {
  constexpr int NT = 128 * DSPLIT;
  constexpr int NS = KEYS ? 2 : BKV / 8;            // key n-tiles a warp forms scores for, per tile
  extern __shared__ __align__(128) unsigned char smem[];
  const int ld = hd + 8;                            // elements per row in shared memory
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* kv_s = q_s + BQ * ld;              // [2][BKV][ld]
  gi::pdl_prologue();

  const int b = blockIdx.z, sp = blockIdx.y;
  const bool decode = cu_seqlens == nullptr;
  const int tok0 = decode ? b : cu_seqlens[b];
  const int qlen = decode ? 1 : cu_seqlens[b + 1] - tok0;
  const int pos0 = decode ? seq_lens[b] - 1 : seq_pos0[b];
  const int R = qlen * n_heads;                     // (token, head) rows of this sequence's step
  // the latest rows of a sequence see the most keys: their blocks start first
  const int rho0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BQ;
  if (rho0 >= R) return;
  const int slot = seq_slots[b];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int wr = KEYS ? 0 : (warp & 3), vh = warp >> 2, wk = warp & 3;
  const int rows_here = min(BQ, R - rho0);
  const int p_last = pos0 + (rho0 + rows_here - 1) / n_heads;
  const int tiles_all = p_last / BKV + 1;
  int tile_lo = 0, tile_hi = tiles_all;
  if (n_splits > 1) {
    const int per = own_tiles > 0 ? own_tiles : (tiles_all + n_splits - 1) / n_splits;
    tile_lo = min(tiles_all, sp * per);
    tile_hi = min(tiles_all, tile_lo + per);
  }
  const int ch = hd / 8;

  auto issue_kv = [&](int tile, int stage) {
    const int kt = tile * BKV;
    const int page = slot >= 0 ? block_table[(size_t)slot * max_pages + kt / PAGE_TOKENS] : 0;
    const __nv_bfloat16* src0 = kcache + (size_t)page * PAGE_TOKENS * dk;
    __nv_bfloat16* ks = kv_s + (size_t)stage * BKV * ld;
    // a warp takes a row at a time, its lanes the row's 16-byte chunks
    for (int r = warp; r < BKV; r += NT / 32) {
      const bool seen = kt + r <= p_last;                            // rows nobody here sees, padding columns: zeros
      for (int c = lane; c < ch; c += 32) {
        const int ok = (seen && c * 8 < dk) ? 16 : 0;
        gi::cp_async_16(gi::smem_u32(ks + r * ld + c * 8), src0 + (ok ? (size_t)r * dk + c * 8 : 0), ok);
      }
    }
  };

  // the queries: only the 16-row groups that hold rows are read by anyone
  for (int r = warp; r < (rows_here + 15) / 16 * 16; r += NT / 32) {
    const int rho = rho0 + r;
    const bool live = r < rows_here;
    const __nv_bfloat16* src0 = q + (live ? (size_t)(tok0 + rho / n_heads) * ldq + (size_t)(rho % n_heads) * dk : 0);
    for (int c = lane; c < ch; c += 32) {
      const int ok = (live && c * 8 < dk) ? 16 : 0;
      gi::cp_async_16(gi::smem_u32(q_s + r * ld + c * 8), src0 + (ok ? c * 8 : 0), ok);
    }
  }
  if (tile_lo < tile_hi) issue_kv(tile_lo, 0);
  gi::cp_async_commit();

  const int r_lo = wr * 16 + g;                                  // this thread's rows: r_lo and r_lo + 8
  const bool ok_row[2] = {r_lo < rows_here, r_lo + 8 < rows_here};
  const int p_row[2] = {pos0 + (rho0 + min(r_lo, rows_here - 1)) / n_heads, pos0 + (rho0 + min(r_lo + 8, rows_here - 1)) / n_heads};
  const bool warp_has_rows = wr * 16 < rows_here;
  const int p_warp_last = pos0 + (rho0 + min(wr * 16 + 15, rows_here - 1)) / n_heads;
  const float sl2 = scale * LOG2E;
  const int dv16 = (dv + 15) / 16 * 16;
  const int vcol0 = vh * NVT * 8;

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[NVT][4];
#pragma unroll
  for (int i = 0; i < NVT; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;

  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    if (tile + 1 < tile_hi) issue_kv(tile + 1, stage ^ 1);
    gi::cp_async_commit();
    gi::cp_async_wait<1>();
    __syncthreads();
    const int kt = tile * BKV;
    const __nv_bfloat16* ks_ = kv_s + (size_t)stage * BKV * ld;
    const int key0 = KEYS ? wk * 16 : 0;                         // first key of the tile this warp looks at
    const bool active = warp_has_rows && kt + key0 <= p_warp_last;
    if (active) {
      float s[NS][4];
#pragma unroll
      for (int nt = 0; nt < NS; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[nt][c] = 0.f;
      if (KEYS) {
        // 16 keys a warp: two chains of products (even and odd slices of the columns) instead of one, added at the end
        float s2[NS][4];
#pragma unroll
        for (int nt = 0; nt < NS; ++nt)
#pragma unroll
          for (int c = 0; c < 4; ++c) s2[nt][c] = 0.f;
        const uint32_t q_at = gi::smem_u32(q_s + ((lane & 7) + ((lane >> 3) & 1) * 8) * ld + (lane >> 4) * 8);
        const uint32_t k_at = gi::smem_u32(ks_ + (key0 + (lane >> 4) * 8 + (lane & 7)) * ld + ((lane >> 3) & 1) * 8);
        const int steps = hd / 16;
        for (int kp = 0; kp + 1 < steps; kp += 2) {
          uint32_t qa_[4], qb_[4], ka_[4], kb_[4];
          gi::ldmatrix_x4(qa_, q_at + kp * 32);
          gi::ldmatrix_x4(ka_, k_at + kp * 32);
          gi::ldmatrix_x4(qb_, q_at + kp * 32 + 32);
          gi::ldmatrix_x4(kb_, k_at + kp * 32 + 32);
          gi::mma_16816(s[0], qa_, ka_[0], ka_[1]);
          gi::mma_16816(s[1], qa_, ka_[2], ka_[3]);
          gi::mma_16816(s2[0], qb_, kb_[0], kb_[1]);
          gi::mma_16816(s2[1], qb_, kb_[2], kb_[3]);
        }
        if (steps & 1) {
          uint32_t qa_[4], ka_[4];
          gi::ldmatrix_x4(qa_, q_at + (steps - 1) * 32);
          gi::ldmatrix_x4(ka_, k_at + (steps - 1) * 32);
          gi::mma_16816(s[0], qa_, ka_[0], ka_[1]);
          gi::mma_16816(s[1], qa_, ka_[2], ka_[3]);
        }
#pragma unroll
        for (int nt = 0; nt < NS; ++nt)
#pragma unroll
          for (int c = 0; c < 4; ++c) s[nt][c] += s2[nt][c];
      } else {
      for (int kp = 0; kp < hd / 16; ++kp) {
        uint32_t qf[4];
        gi::ldmatrix_x4(qf, gi::smem_u32(q_s + (wr * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * ld + (kp * 2 + (lane >> 4)) * 8));
#pragma unroll
        for (int n2 = 0; n2 < NS / 2; ++n2) {
          uint32_t kb[4];
          const int r = key0 + (n2 * 2 + (lane >> 4)) * 8 + (lane & 7);
          gi::ldmatrix_x4(kb, gi::smem_u32(ks_ + r * ld + (kp * 2 + ((lane >> 3) & 1)) * 8));
          gi::mma_16816(s[n2 * 2], qf, kb[0], kb[1]);
          gi::mma_16816(s[n2 * 2 + 1], qf, kb[2], kb[3]);
        }
      }
      }
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < NS; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = kt + key0 + nt * 8 + 2 * t + (c & 1);
          const bool ok = ok_row[c >> 1] && key <= p_row[c >> 1];
          s[nt][c] = ok ? s[nt][c] * sl2 : -INFINITY;
          tmax[c >> 1] = fmaxf(tmax[c >> 1], s[nt][c]);
        }
      float alpha[2], m_use[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 1));
        tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 2));
        const float m_new = fmaxf(m_run[hh], tmax[hh]);
        alpha[hh] = (m_run[hh] == -INFINITY) ? 0.f : exp2f(m_run[hh] - m_new);
        m_run[hh] = m_new;
        m_use[hh] = (m_new == -INFINITY) ? 0.f : m_new;
      }
      float psum[2] = {0.f, 0.f};
      uint32_t pf[NS / 2][4];
#pragma unroll
      for (int nt = 0; nt < NS; ++nt) {
        const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
        const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
        psum[0] += p0 + p1;
        psum[1] += p2 + p3;
        pf[nt / 2][(nt & 1) * 2] = gi::pack_bf16(p0, p1);
        pf[nt / 2][(nt & 1) * 2 + 1] = gi::pack_bf16(p2, p3);
      }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 1);
        psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 2);
        l_run[hh] = l_run[hh] * alpha[hh] + psum[hh];
      }
#pragma unroll
      for (int i = 0; i < NVT; ++i) {
        o[i][0] *= alpha[0];
        o[i][1] *= alpha[0];
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
#pragma unroll
      for (int kk = 0; kk < NS / 2; ++kk) {
#pragma unroll
        for (int dp = 0; dp < NVT / 2; ++dp) {
          if (vcol0 + dp * 16 < dv16) {            // the same for the whole warp
            uint32_t vb[4];
            const int r = key0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            gi::ldmatrix_x4_trans(vb, gi::smem_u32(ks_ + r * ld + vcol0 + (dp * 2 + (lane >> 4)) * 8));
            gi::mma_16816(o[dp * 2], pf[kk], vb[0], vb[1]);
            gi::mma_16816(o[dp * 2 + 1], pf[kk], vb[2], vb[3]);
          }
        }
      }
    }
    __syncthreads();     // everyone is done with this stage before the next iteration refills it
  }
  gi::cp_async_wait<0>();

  if (!KEYS) {
#pragma unroll
    for (int hh = 0; hh < 2; ++hh) {
      const int row = r_lo + hh * 8;
      if (row >= rows_here) continue;
      const int rho = rho0 + row;
      const int tokl = rho / n_heads, head = rho % n_heads;
      if (n_splits == 1) {
        const float inv = l_run[hh] > 0.f ? 1.0f / l_run[hh] : 0.f;
        __nv_bfloat16* orow = out + (size_t)(tok0 + tokl) * ldo + (size_t)head * dv;
#pragma unroll
        for (int i = 0; i < NVT; ++i) {
          const int col = vcol0 + i * 8 + 2 * t;
          if (col < dv)
            *reinterpret_cast<__nv_bfloat162*>(orow + col) = __floats2bfloat162_rn(o[i][hh * 2] * inv, o[i][hh * 2 + 1] * inv);
        }
      } else {
        const size_t pi = ((size_t)b * n_heads + head) * n_splits + sp;
#pragma unroll
        for (int i = 0; i < NVT; ++i) {
          const int col = vcol0 + i * 8 + 2 * t;
          if (col < dv) *reinterpret_cast<float2*>(part_o + pi * dv + col) = make_float2(o[i][hh * 2], o[i][hh * 2 + 1]);
        }
        if (t == 0 && vh == 0) {
          part_ml[pi * 2] = m_run[hh] == -INFINITY ? -INFINITY : m_run[hh] * LN2;
          part_ml[pi * 2 + 1] = l_run[hh];
        }
      }
    }
    return;
  }

  // keys mode: the warps' statistics and outputs meet in shared memory (the tiles are not needed any more)
  constexpr int MO_LD = NVT * 8 + 8;                              // rows 8 floats longer: the warps' stores meet fewer banks twice
  float* mo = reinterpret_cast<float*>(smem);                     // [warps][16][MO_LD]
  float* mm = mo + (size_t)4 * DSPLIT * 16 * MO_LD;              // [warps][16] maxima (base 2), then [warps][16] sums
  float* ml = mm + 4 * DSPLIT * 16;
#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int row = g + hh * 8;
    if (t == 0) {
      mm[warp * 16 + row] = m_run[hh];
      ml[warp * 16 + row] = l_run[hh];
    }
#pragma unroll
    for (int i = 0; i < NVT; ++i) {
      *reinterpret_cast<float2*>(mo + ((size_t)warp * 16 + row) * MO_LD + i * 8 + 2 * t) = make_float2(o[i][hh * 2], o[i][hh * 2 + 1]);
    }
  }
  __syncthreads();
  // sixteen threads a row: a row's weights are worked out once, then its columns are walked
  {
    const int row = tid >> 4, c0 = tid & 15;
    if (row < rows_here) {                       // NT / 16 >= 8 rows a pass; rows_here <= 16
      for (int rr = row; rr < rows_here; rr += NT / 16) {
        const int rho = rho0 + rr;
        const int tokl = rho / n_heads, head = rho % n_heads;
        const size_t pi = ((size_t)b * n_heads + head) * n_splits + sp;
        for (int half = 0; half < DSPLIT; ++half) {
          float mx = -INFINITY;
#pragma unroll
          for (int w = 0; w < 4; ++w) mx = fmaxf(mx, mm[(half * 4 + w) * 16 + rr]);
          float wgt[4], tot = 0.f;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            const float mw = mm[(half * 4 + w) * 16 + rr];
            wgt[w] = (mx == -INFINITY || mw == -INFINITY) ? 0.f : exp2f(mw - mx);
            tot += ml[(half * 4 + w) * 16 + rr] * wgt[w];
          }
          const float inv = tot > 0.f ? 1.0f / tot : 0.f;
          const int col_end = min(dv, (half + 1) * NVT * 8);
          for (int col = half * NVT * 8 + c0; col < col_end; col += 16) {
            const int cin = col - half * NVT * 8;
            float val = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) val += mo[((size_t)(half * 4 + w) * 16 + rr) * MO_LD + cin] * wgt[w];
            if (n_splits == 1) out[(size_t)(tok0 + tokl) * ldo + (size_t)head * dv + col] = __float2bfloat16_rn(val * inv);
            else part_o[pi * dv + col] = val;
          }
          if (n_splits > 1 && half == 0 && c0 == 0) {
            part_ml[pi * 2] = mx == -INFINITY ? -INFINITY : mx * LN2;
            part_ml[pi * 2 + 1] = tot;
          }
        }
      }
    }
  }
}

template <int NVT, int DSPLIT, bool KEYS>
int launch(dim3 grid, size_t smem, cudaStream_t s, __nv_bfloat16* out, long ldo, float* po, float* pml, const __nv_bfloat16* q, long ldq,
           const __nv_bfloat16* kc, const int* bt, int max_pages, const int* cu, const int* slots, const int* pos0, const int* lens, int H,
           float scale, int dk, int dv, int hd, int n_splits, int own_tiles) {
  auto kern = attn_latent_mma_kernel<NVT, DSPLIT, KEYS>;
  if (KEYS) smem = max(smem, (size_t)4 * DSPLIT * 16 * (NVT * 8 + 8 + 2) * sizeof(float));
  static size_t configured[gi::MAX_DEVICES_SEEN] = {0};
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= gi::MAX_DEVICES_SEEN) dev = -1;
  if (smem > 48 * 1024 && (dev < 0 || configured[dev] < smem)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "latent attention: %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = smem;
  }
  cudaError_t e = gi::launch(kern, grid, dim3(128 * DSPLIT), smem, s, out, ldo, po, pml, q, ldq, kc, bt, max_pages, cu, slots, pos0,
                             lens, H, scale, dk, dv, hd, n_splits, own_tiles);
  return gi::check(e, "latent attention (tensor cores)");
}

}  // namespace

// cu_seqlens null: a one-token step (seq_lens gives the lengths including the step's token; n_splits slices, merged here).
extern "C" int gi_attn_latent_tc(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                                 const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                                 const int* seq_pos0, const int* seq_lens, int n_seqs, int max_q_len, int n_heads, int dk, int dv,
                                 float scale, int n_splits, int own_tiles, void* stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return GI_OK;
  if (dk <= 0 || dk > 576 || dk % 8 || dv <= 0 || dv > 512 || dv % 8 || dv > dk)
    return gi::fail(GI_ERR_UNSUPPORTED, "latent attention (tensor cores): rows of %d with values of %d; multiples of 8 up to 576 and 512", dk, dv);
  if (ldq % 8 != 0 || ldo % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kcache & 15) || ((uintptr_t)out & 3))
    return gi::fail(GI_ERR_UNSUPPORTED, "latent attention (tensor cores): queries and cache must be 16-byte aligned");
  const bool decode = cu_seqlens == nullptr;
  if (decode ? (seq_lens == nullptr || max_q_len != 1) : (seq_pos0 == nullptr || n_splits != 1))
    return gi::fail(GI_ERR_ARG, "latent attention: a one-token step needs lengths, a prompt step start positions and one slice");
  if (n_splits < 1 || (n_splits > 1 && (!part_o || !part_ml))) return gi::fail(GI_ERR_ARG, "latent attention: slices need scratch memory");
  const long q_tiles = ((long)max_q_len * n_heads + BQ - 1) / BQ;
  if (n_seqs > 65535 || n_splits > 65535 || q_tiles > 0x7fffffffL) return gi::fail(GI_ERR_UNSUPPORTED, "latent attention: too many sequences, slices or rows for one launch");
  const int hd = (dk + 15) / 16 * 16, dv16 = (dv + 15) / 16 * 16;
  const size_t smem = (size_t)3 * BQ * (hd + 8) * 2;
  dim3 grid((unsigned)q_tiles, n_splits, n_seqs);
  cudaStream_t s = (cudaStream_t)stream;
  const bool keys = decode && n_heads <= 16;
  int rc;
#define GI_LAT(NVT, DS)                                                                                                          \
  rc = keys ? launch<NVT, DS, true>(grid, smem, s, (__nv_bfloat16*)out, ldo, part_o, part_ml, (const __nv_bfloat16*)q, ldq,       \
                                    (const __nv_bfloat16*)kcache, block_table, max_pages, cu_seqlens, seq_slots, seq_pos0, seq_lens, \
                                    n_heads, scale, dk, dv, hd, n_splits, own_tiles)                                             \
            : launch<NVT, DS, false>(grid, smem, s, (__nv_bfloat16*)out, ldo, part_o, part_ml, (const __nv_bfloat16*)q, ldq,      \
                                     (const __nv_bfloat16*)kcache, block_table, max_pages, cu_seqlens, seq_slots, seq_pos0, seq_lens, \
                                     n_heads, scale, dk, dv, hd, n_splits, own_tiles)
  if (dv16 <= 64) { GI_LAT(8, 1); }
  else if (dv16 <= 128) { GI_LAT(16, 1); }
  else if (dv16 <= 256) { GI_LAT(32, 1); }
  else { GI_LAT(32, 2); }
#undef GI_LAT
  if (rc != GI_OK) return rc;
  if (n_splits > 1) return gi_attn_combine(out, ldo, GI_BF16, part_o, part_ml, n_seqs, n_heads, dv, n_splits, stream);
  return GI_OK;
}
