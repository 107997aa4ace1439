// Causal attention over a paged latent cache, in the absorbed form: every head of a token scores against the
// same cached row [ latent c (R) | rotated shared key part (P) ] and sums the latents c themselves,
//
//   s_j  = ( q_lat[t, h, :R] . c_j  +  q_lat[t, h, R:] . kr_j ) * scale        for the visible j
//   o_lat[t, h, :] = sum_j softmax(s)_j c_j                                     [R]
//
// where q_lat[t, h, :R] = W_uk[h]^T q_unrotated is made by the product before this kernel and the product behind
// it applies W_uv[h] to o_lat.  One row of the cache serves as key and as value for all heads (multi-query
// attention with a key of R + P and a value of R elements).  Scores, softmax and sums are 32-bit.
//
// This file: the plain-arithmetic kernel (any R, P; f32 or bf16 storage): one warp per (token, head), keys
// visited four at a time in position order with an online softmax, `expf`.  It is the whole attention of the
// 32-bit engine and the fallback of the bfloat16 engine for sizes the tensor-core kernel refuses.
#include "common.cuh"

using namespace dinfer;

namespace {

constexpr int WARPS = 4;
constexpr int KEYS = 4;

template <typename T, int C>   // C = ceil((R + P) / 32) elements per lane
__global__ void __launch_bounds__(WARPS * 32)
attention_latent_generic_kernel(const T* __restrict__ q, int64_t ldq_t, int64_t ldq_h, T* __restrict__ out,
                                int64_t ldo_t, int64_t ldo_h, const T* __restrict__ cache,
                                const int* __restrict__ block_table, int max_blocks,
                                const int* __restrict__ cu_seqlens, const int* __restrict__ positions, int num_reqs,
                                int H, int R, int P, int block_size, float scale, int window) {
  pdl_enter();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * WARPS + warp;
  if (h >= H) return;
  int lo = 0, hi = num_reqs - 1;                         // request of this token: last b with cu_seqlens[b] <= t
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_seqlens[mid] <= t) lo = mid; else hi = mid - 1;
  }
  const int* table = block_table + (int64_t)lo * max_blocks;
  const int pos = positions[t];
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int W = R + P;

  float qv[C], acc[C];
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int e = lane + 32 * c;
    qv[c] = e < W ? to_f32<T>(q[(int64_t)t * ldq_t + (int64_t)h * ldq_h + e]) * scale : 0.f;
    acc[c] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int j0 = first; j0 <= pos; j0 += KEYS) {
    const T* kp[KEYS];
    float s[KEYS];
#pragma unroll
    for (int u = 0; u < KEYS; ++u) {
      const int j = j0 + u;
      kp[u] = nullptr;
      s[u] = 0.f;
      const int64_t blk = j <= pos ? table[j / block_size] : -1;       // -1: a page the table does not hold is no key
      if (blk >= 0) {
        kp[u] = cache + (blk * block_size + j % block_size) * W;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int e = lane + 32 * c;
          if (e < W) s[u] += qv[c] * to_f32<T>(kp[u][e]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < KEYS; ++u) s[u] = kp[u] ? warp_sum(s[u]) : -INFINITY;
    float m_new = m;
#pragma unroll
    for (int u = 0; u < KEYS; ++u) m_new = fmaxf(m_new, s[u]);
    if (m_new == -INFINITY) continue;
    const float alpha = expf(m - m_new);
    l *= alpha;
#pragma unroll
    for (int c = 0; c < C; ++c) acc[c] *= alpha;
#pragma unroll
    for (int u = 0; u < KEYS; ++u) {
      if (kp[u]) {
        const float p = expf(s[u] - m_new);
        l += p;
#pragma unroll
        for (int c = 0; c < C; ++c) {
          const int e = lane + 32 * c;
          if (e < R) acc[c] += p * to_f32<T>(kp[u][e]);
        }
      }
    }
    m = m_new;
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
  for (int c = 0; c < C; ++c) {
    const int e = lane + 32 * c;
    if (e < R) out[(int64_t)t * ldo_t + (int64_t)h * ldo_h + e] = from_f32<T>(acc[c] * inv);
  }
}

template <typename T, int C>
int launch_generic(const void* q, int64_t ldq_t, int64_t ldq_h, void* out, int64_t ldo_t, int64_t ldo_h,
                   const void* cache, const int* block_table, int max_blocks, const int* cu_seqlens,
                   const int* positions, int T_, int B, int H, int R, int P, int block_size, float scale, int window,
                   cudaStream_t stream) {
  dim3 grid(T_, (H + WARPS - 1) / WARPS);
  launch_pdl(attention_latent_generic_kernel<T, C>, grid, dim3(WARPS * 32), 0, stream, (const T*)q, ldq_t, ldq_h,
             (T*)out, ldo_t, ldo_h, (const T*)cache, block_table, max_blocks, cu_seqlens, positions, B, H, R, P,
             block_size, scale, window);
  return cuda_status("attention_latent_generic");
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// q [T, H, R + P] with element strides (ldq_t, ldq_h); out [T, H, R] with (ldo_t, ldo_h); cache
// [pages, block_size, R + P] contiguous; block_table [B, max_blocks] int32; cu_seqlens [B + 1]; positions [T].
// window <= 0: all keys.
DINFER_API int dinfer_attention_latent_generic(const void* q, int64_t ldq_t, int64_t ldq_h, void* out, int64_t ldo_t,
                                               int64_t ldo_h, const void* cache, const int* block_table,
                                               int max_blocks, const int* cu_seqlens, const int* positions, int T,
                                               int B, int H, int R, int P, int block_size, float scale, int window,
                                               int dtype, cudaStream_t stream) {
  if (T < 0 || B <= 0 || H <= 0 || R <= 0 || P < 0 || block_size <= 0 || max_blocks <= 0)
    return refuse(DINFER_BAD_ARGUMENT, "attention_latent_generic: bad sizes T=%d B=%d H=%d R=%d P=%d block=%d", T, B, H,
                  R, P, block_size);
  if (R + P > 1024) return refuse(DINFER_BAD_ARGUMENT, "attention_latent_generic: row of %d above the limit 1024", R + P);
  if ((H + WARPS - 1) / WARPS > 65535) return refuse(DINFER_BAD_ARGUMENT, "attention_latent_generic: too many heads");
  if (T == 0) return 0;
  const int c = (R + P + 31) / 32;
#define GO(C) return launch_generic<T_, C>(q, ldq_t, ldq_h, out, ldo_t, ldo_h, cache, block_table, max_blocks, \
                                           cu_seqlens, positions, T, B, H, R, P, block_size, scale, window, stream)
  DINFER_DISPATCH_DTYPE(dtype, T_, {
    if (c <= 1) GO(1);
    else if (c <= 2) GO(2);
    else if (c <= 3) GO(3);
    else if (c <= 4) GO(4);
    else if (c <= 6) GO(6);
    else if (c <= 8) GO(8);
    else if (c <= 12) GO(12);
    else if (c <= 18) GO(18);
    else GO(32);
  });
#undef GO
  return 0;
}
