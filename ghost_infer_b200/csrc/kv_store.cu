// Keys and values of a step's tokens into the paged cache for an attention without rotation, whose values may have
// another width than its keys and may first be blended with the values another layer computed for the same tokens:
// v <- (1 - lambda) v + lambda v_first, in 32-bit, lambda a learned scalar read from device memory.
// Rows are packed [q: heads * hd | k: kv * hd | v: kv * hdv]; the cache is keys [page][kv head][64][hd] and values
// [page][kv head][64][hdv].  Padding rows (slot -1) land on the trash page 0.
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void kv_store_kernel(T* qkv, long ld, const T* first, const float* __restrict__ lambda, T* copy_to,
                                const int* __restrict__ positions, const int* __restrict__ slots,
                                const int* __restrict__ block_table, int max_pages, T* __restrict__ kcache,
                                T* __restrict__ vcache, int n_heads, int n_kv, int hd, int hdv, int write_cache) {
  gi::pdl_prologue();
  const int t = blockIdx.x;
  const int pos = positions[t], slot = slots[t];
  const int page = (write_cache && slot >= 0) ? block_table[(size_t)slot * max_pages + pos / PAGE_TOKENS] : 0;
  const int off = pos % PAGE_TOKENS;
  T* row = qkv + (size_t)t * ld;
  const int kw = n_kv * hd, vw = n_kv * hdv;
  if (write_cache) {
    for (int i = threadIdx.x; i < kw; i += blockDim.x) {
      const int g = i / hd, d = i % hd;
      kcache[(((size_t)page * n_kv + g) * PAGE_TOKENS + off) * hd + d] = row[(size_t)n_heads * hd + i];
    }
  }
  const float lam = (first != nullptr) ? *lambda : 0.f;
  for (int i = threadIdx.x; i < vw; i += blockDim.x) {
    T* vp = row + (size_t)n_heads * hd + kw + i;
    T val = *vp;
    if (copy_to != nullptr) copy_to[(size_t)t * vw + i] = val;
    if (first != nullptr) {
      const float mixed = (1.0f - lam) * gi::ldf(vp) + lam * gi::ldf(first + (size_t)t * vw + i);
      gi::stf(vp, mixed);
      val = *vp;
    }
    if (write_cache) {
      const int g = i / hdv, d = i % hdv;
      vcache[(((size_t)page * n_kv + g) * PAGE_TOKENS + off) * hdv + d] = val;
    }
  }
}

}  // namespace

extern "C" int gi_kv_store(void* qkv, int dtype, long ld, const void* first, const float* lambda, void* copy_to,
                           const int* positions, const int* slots, const int* block_table, int max_pages, void* kcache,
                           void* vcache, int n_tokens, int n_heads, int n_kv, int hd, int hdv, int write_cache,
                           void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (n_heads <= 0 || n_kv <= 0 || hd <= 0 || hdv <= 0) return gi::fail(GI_ERR_ARG, "kv store: bad sizes");
  if (first != nullptr && lambda == nullptr) return gi::fail(GI_ERR_ARG, "kv store: blending needs its weight");
  if (write_cache && (!kcache || !vcache || !block_table)) return gi::fail(GI_ERR_ARG, "kv store: cache write without a cache");
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(kv_store_kernel<T>, dim3(n_tokens), dim3(128), 0, (cudaStream_t)stream, (T*)qkv, ld, (const T*)first, lambda,
                     (T*)copy_to, positions, slots, block_table, max_pages, (T*)kcache, (T*)vcache, n_heads, n_kv, hd, hdv,
                     write_cache));
  return gi::check(e, "kv store");
}
