// RMSNorm over rows of the 32-bit residual stream, with the residual add and the row gather
// fused in.  One block per output row.
//
//   v      = residual[src] + delta[src]          (delta optional; src = rows[r] or r)
//   residual[src] = v                            (only when delta is given and rows is not)
//   out[r] = T( v * rsqrt(mean(v^2) + eps) * w ) (one rounding, after the weight multiply)
//
// Sum of squares, rsqrt and products are 32-bit.  Counterpart in the reference:
// crates/kernels/cuda/norm.cu:41-116 (rmsnorm / fused_add_rmsnorm / gather_rmsnorm), which keeps
// the residual in bf16; here it stays in 32-bit so that the sum is exact to rounding of one add.
#include "common.cuh"

using namespace dinfer;

namespace {

// four consecutive elements at once (16 bytes of f32, 8 bytes of bf16)
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&v)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 x = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&v)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&v)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&v)[4]) {
  uint2 x;
  *reinterpret_cast<__nv_bfloat162*>(&x.x) = __floats2bfloat162_rn(v[0], v[1]);
  *reinterpret_cast<__nv_bfloat162*>(&x.y) = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = x;
}

template <typename TA, typename TW, int VEC>
__global__ void __launch_bounds__(1024)
rmsnorm_kernel(float* __restrict__ residual, const TA* __restrict__ delta, const int* __restrict__ rows,
               const TW* __restrict__ weight, TA* __restrict__ out, int h, float eps, int stash) {
  extern __shared__ float sm_row[];
  __shared__ float red[33];
  pdl_enter();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (int64_t)src * h;
  const TA* del = delta ? delta + (int64_t)src * h : nullptr;
  const bool writeback = (delta != nullptr) && (rows == nullptr);
  TA* o = out + (int64_t)r * h;

  float ss = 0.f;
  for (int i = threadIdx.x * VEC; i < h; i += blockDim.x * VEC) {
    float v[4];
    if (VEC == 4) {
      load4<float>(res + i, v);
      if (del) {
        float d[4];
        load4<TA>(del + i, d);
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += d[j];
        if (writeback) store4<float>(res + i, v);
      }
    } else {
      v[0] = res[i];
      if (del) {
        v[0] += to_f32<TA>(del[i]);
        if (writeback) res[i] = v[0];
      }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      ss += v[j] * v[j];
      if (stash) sm_row[i + j] = v[j];
    }
  }
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)h + eps);
  for (int i = threadIdx.x * VEC; i < h; i += blockDim.x * VEC) {
    float v[4], w[4];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      if (stash) v[j] = sm_row[i + j];
      else v[j] = res[i + j] + ((del && !writeback) ? to_f32<TA>(del[i + j]) : 0.f);
    }
    if (VEC == 4) {
      load4<TW>(weight + i, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = v[j] * rinv * w[j];
      store4<TA>(o + i, v);
    } else {
      o[i] = from_f32<TA>(v[0] * rinv * to_f32<TW>(weight[i]));
    }
  }
}

template <typename TA, typename TW>
int launch(float* residual, const void* delta, const int* rows, const void* weight, void* out,
           int num_rows, int h, float eps, cudaStream_t stream) {
  if (num_rows == 0) return 0;
  const auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec4 = (h % 4 == 0) && al(residual) && al(delta) && al(weight) && al(out);
  const int per = vec4 ? 4 : 1;
  int threads = (h / per + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  const size_t row_bytes = (size_t)h * sizeof(float);
  const int stash = row_bytes <= 64 * 1024;
  const size_t smem = stash ? row_bytes : 0;
  auto k4 = rmsnorm_kernel<TA, TW, 4>;
  auto k1 = rmsnorm_kernel<TA, TW, 1>;
  auto k = vec4 ? k4 : k1;
  static bool opted[2] = {false, false};   // once per process and kernel, kept out of graph captures
  if (smem > 48 * 1024 && !opted[vec4]) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return refuse((int)e, "rmsnorm: shared memory opt-in failed: %s", cudaGetErrorString(e));
    opted[vec4] = true;
  }
  launch_pdl(k, dim3(num_rows), dim3(threads), smem, stream, residual, (const TA*)delta, rows, (const TW*)weight, (TA*)out, h, eps, stash);
  return cuda_status("rmsnorm");
}

// Plain RMSNorm of rows that are not the residual stream (toy parts, tests): x of type TA.
template <typename TA, typename TW>
__global__ void rmsnorm_plain_kernel(const TA* __restrict__ x, const TW* __restrict__ weight,
                                     TA* __restrict__ out, int h, float eps) {
  __shared__ float red[33];
  const TA* row = x + (int64_t)blockIdx.x * h;
  float ss = 0.f;
  for (int i = threadIdx.x; i < h; i += blockDim.x) { const float v = to_f32<TA>(row[i]); ss += v * v; }
  ss = block_sum(ss, red);
  const float rinv = rsqrtf(ss / (float)h + eps);
  for (int i = threadIdx.x; i < h; i += blockDim.x)
    out[(int64_t)blockIdx.x * h + i] = from_f32<TA>(to_f32<TA>(row[i]) * rinv * to_f32<TW>(weight[i]));
}


// Layer norm (weight and bias) over rows of the 32-bit residual stream, with up to two pending branch outputs
// added first, each times a per-channel scale, and up to two normed outputs of the same row (two norms with their
// own weights: the layers whose mixer and feed-forward read the same x):
//
//   v      = residual[src] + d1[src] * s1 + d2[src] * s2      (each optional; s null = 1; src = rows[r] or r)
//   residual[src] = v                                         (when a delta is given and rows is not)
//   mu = mean(v), var = mean((v - mu)^2)                      (two passes over the row kept in shared memory)
//   out_k[r] = T( (v - mu) * rsqrt(var + eps) * w_k + b_k )   (k = 1, 2; b null = 0)
template <typename TA, typename TW>
__global__ void __launch_bounds__(1024)
layernorm_kernel(float* __restrict__ residual, const TA* __restrict__ d1, const TW* __restrict__ s1,
                 const TA* __restrict__ d2, const TW* __restrict__ s2, const int* __restrict__ rows,
                 const TW* __restrict__ w1, const TW* __restrict__ b1, TA* __restrict__ out1,
                 const TW* __restrict__ w2, const TW* __restrict__ b2, TA* __restrict__ out2, int h, float eps,
                 int stash) {
  extern __shared__ float sm_row[];
  __shared__ float red[33];
  pdl_enter();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (int64_t)src * h;
  const TA* e1 = d1 ? d1 + (int64_t)src * h : nullptr;
  const TA* e2 = d2 ? d2 + (int64_t)src * h : nullptr;
  const bool writeback = (e1 || e2) && rows == nullptr;
  auto value = [&](int i) {
    float v = res[i];
    if (e1) v += to_f32<TA>(e1[i]) * (s1 ? to_f32<TW>(s1[i]) : 1.f);
    if (e2) v += to_f32<TA>(e2[i]) * (s2 ? to_f32<TW>(s2[i]) : 1.f);
    return v;
  };
  float sum = 0.f;
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    const float v = value(i);
    if (stash) sm_row[i] = v;
    sum += v;
  }
  const float mu = block_sum(sum, red) / (float)h;
  float sq = 0.f;
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    const float d = (stash ? sm_row[i] : value(i)) - mu;
    sq += d * d;
  }
  const float rinv = rsqrtf(block_sum(sq, red) / (float)h + eps);
  for (int i = threadIdx.x; i < h; i += blockDim.x) {
    const float v = stash ? sm_row[i] : value(i);
    const float n = (v - mu) * rinv;
    out1[(int64_t)r * h + i] = from_f32<TA>(n * to_f32<TW>(w1[i]) + (b1 ? to_f32<TW>(b1[i]) : 0.f));
    if (out2) out2[(int64_t)r * h + i] = from_f32<TA>(n * to_f32<TW>(w2[i]) + (b2 ? to_f32<TW>(b2[i]) : 0.f));
    if (writeback) res[i] = v;           // after every read of the old value by this thread (same i, same thread)
  }
}

// The same with four consecutive elements per thread and step (h a multiple of 4, every pointer 16-byte aligned, the
// row kept in shared memory): 16-byte loads of the residual, 8-byte ones of bfloat16 operands.
template <typename TA, typename TW>
__global__ void __launch_bounds__(1024)
layernorm_vec4_kernel(float* __restrict__ residual, const TA* __restrict__ d1, const TW* __restrict__ s1,
                      const TA* __restrict__ d2, const TW* __restrict__ s2, const int* __restrict__ rows,
                      const TW* __restrict__ w1, const TW* __restrict__ b1, TA* __restrict__ out1,
                      const TW* __restrict__ w2, const TW* __restrict__ b2, TA* __restrict__ out2, int h, float eps) {
  extern __shared__ float sm_row[];
  __shared__ float red[33];
  pdl_enter();
  const int r = blockIdx.x;
  const int src = rows ? rows[r] : r;
  float* res = residual + (int64_t)src * h;
  const TA* e1 = d1 ? d1 + (int64_t)src * h : nullptr;
  const TA* e2 = d2 ? d2 + (int64_t)src * h : nullptr;
  const bool writeback = (e1 || e2) && rows == nullptr;
  float sum = 0.f;
  for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
    float v[4], d[4], s[4];
    load4<float>(res + i, v);
    if (e1) {
      load4<TA>(e1 + i, d);
      if (s1) { load4<TW>(s1 + i, s); }
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] += d[j] * (s1 ? s[j] : 1.f);
    }
    if (e2) {
      load4<TA>(e2 + i, d);
      if (s2) { load4<TW>(s2 + i, s); }
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] += d[j] * (s2 ? s[j] : 1.f);
    }
    if (writeback) store4<float>(res + i, v);
#pragma unroll
    for (int j = 0; j < 4; ++j) { sm_row[i + j] = v[j]; sum += v[j]; }
  }
  const float mu = block_sum(sum, red) / (float)h;
  float sq = 0.f;
  for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
#pragma unroll
    for (int j = 0; j < 4; ++j) { const float d = sm_row[i + j] - mu; sq += d * d; }
  }
  const float rinv = rsqrtf(block_sum(sq, red) / (float)h + eps);
  for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
    float n[4], w[4], b[4], o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) n[j] = (sm_row[i + j] - mu) * rinv;
    load4<TW>(w1 + i, w);
    if (b1) { load4<TW>(b1 + i, b); }
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = n[j] * w[j] + (b1 ? b[j] : 0.f);
    store4<TA>(out1 + (int64_t)r * h + i, o);
    if (out2) {
      load4<TW>(w2 + i, w);
      if (b2) { load4<TW>(b2 + i, b); }
#pragma unroll
      for (int j = 0; j < 4; ++j) o[j] = n[j] * w[j] + (b2 ? b[j] : 0.f);
      store4<TA>(out2 + (int64_t)r * h + i, o);
    }
  }
}

// residual += d1 * s1 + d2 * s2 for rows nobody norms (a pending sum resolved on its own)
template <typename TA, typename TW>
__global__ void scaled_add_kernel(float* __restrict__ residual, const TA* __restrict__ d1, const TW* __restrict__ s1,
                                  const TA* __restrict__ d2, const TW* __restrict__ s2, int64_t n, int h) {
  pdl_enter();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % h);
    float v = residual[i];
    if (d1) v += to_f32<TA>(d1[i]) * (s1 ? to_f32<TW>(s1[c]) : 1.f);
    if (d2) v += to_f32<TA>(d2[i]) * (s2 ? to_f32<TW>(s2[c]) : 1.f);
    residual[i] = v;
  }
}

}  // namespace

DINFER_DEFINE_LAST_ERROR()

// residual [*, h] f32 (updated in place when delta is given and rows is null); delta [*, h] act
// dtype or null; rows [num_rows] int32 or null; weight [h]; out [num_rows, h] act dtype.
DINFER_API int dinfer_rmsnorm(float* residual, const void* delta, const int* rows, const void* weight,
                              void* out, int num_rows, int h, float eps, int act_dtype, int w_dtype,
                              cudaStream_t stream) {
  if (h <= 0 || num_rows < 0) return refuse(DINFER_BAD_ARGUMENT, "rmsnorm: bad sizes rows=%d h=%d", num_rows, h);
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW,
      return launch<TA, TW>(residual, delta, rows, weight, out, num_rows, h, eps, stream)));
  return 0;
}

DINFER_API int dinfer_rmsnorm_plain(const void* x, const void* weight, void* out, int num_rows, int h,
                                    float eps, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (h <= 0 || num_rows < 0) return refuse(DINFER_BAD_ARGUMENT, "rmsnorm_plain: bad sizes rows=%d h=%d", num_rows, h);
  if (num_rows == 0) return 0;
  int threads = (h + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      rmsnorm_plain_kernel<TA, TW><<<num_rows, threads, 0, stream>>>((const TA*)x, (const TW*)weight, (TA*)out, h, eps);
      return cuda_status("rmsnorm_plain");
    }));
  return 0;
}

// residual [*, h] f32 (updated in place when a delta is given and rows is null); d1, d2 [*, h] act dtype or null with
// their per-channel scales s1, s2 [h] (null: 1); rows [num_rows] int32 or null; w1, b1 (and w2, b2 with out2) [h];
// out1, out2 [num_rows, h] act dtype (out2 null: one norm).
DINFER_API int dinfer_layernorm(float* residual, const void* d1, const void* s1, const void* d2, const void* s2,
                                const int* rows, const void* w1, const void* b1, void* out1, const void* w2,
                                const void* b2, void* out2, int num_rows, int h, float eps, int act_dtype,
                                int w_dtype, cudaStream_t stream) {
  if (h <= 0 || num_rows < 0) return refuse(DINFER_BAD_ARGUMENT, "layernorm: bad sizes rows=%d h=%d", num_rows, h);
  if (!w1 || !out1 || (out2 && !w2)) return refuse(DINFER_BAD_ARGUMENT, "layernorm: an output without its weight");
  if (num_rows == 0) return 0;
  int threads = (h + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  const size_t row_bytes = (size_t)h * sizeof(float);
  const int stash = row_bytes <= 48 * 1024;
  const auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  if (stash && h % 4 == 0 && al(residual) && al(d1) && al(s1) && al(d2) && al(s2) && al(w1) && al(b1) && al(out1) && al(w2) &&
      al(b2) && al(out2)) {
    int t4 = (h / 4 + 31) / 32 * 32;
    if (t4 > 512) t4 = 512;
    DINFER_DISPATCH_DTYPE(act_dtype, TA,
      DINFER_DISPATCH_DTYPE(w_dtype, TW, {
        launch_pdl(layernorm_vec4_kernel<TA, TW>, dim3(num_rows), dim3(t4), row_bytes, stream, residual, (const TA*)d1,
                   (const TW*)s1, (const TA*)d2, (const TW*)s2, rows, (const TW*)w1, (const TW*)b1, (TA*)out1,
                   (const TW*)w2, (const TW*)b2, (TA*)out2, h, eps);
        return cuda_status("layernorm");
      }));
  }
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      launch_pdl(layernorm_kernel<TA, TW>, dim3(num_rows), dim3(threads), stash ? row_bytes : 0, stream, residual,
                 (const TA*)d1, (const TW*)s1, (const TA*)d2, (const TW*)s2, rows, (const TW*)w1, (const TW*)b1,
                 (TA*)out1, (const TW*)w2, (const TW*)b2, (TA*)out2, h, eps, stash);
      return cuda_status("layernorm");
    }));
  return 0;
}

DINFER_API int dinfer_scaled_add(float* residual, const void* d1, const void* s1, const void* d2, const void* s2,
                                 int num_rows, int h, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (h <= 0 || num_rows < 0) return refuse(DINFER_BAD_ARGUMENT, "scaled_add: bad sizes rows=%d h=%d", num_rows, h);
  if (num_rows == 0 || (!d1 && !d2)) return 0;
  const int64_t n = (int64_t)num_rows * h;
  const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
  DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      launch_pdl(scaled_add_kernel<TA, TW>, dim3(blocks), dim3(256), 0, stream, residual, (const TA*)d1,
                 (const TW*)s1, (const TA*)d2, (const TW*)s2, n, h);
      return cuda_status("scaled_add");
    }));
  return 0;
}

// A branch output that is normed before it joins the residual stream (a layer with its norm on the sublayer's
// output), and the mean of two branches that are each normed first (two mixers side by side):
//
//   y      = a                                   one branch, no inner norm (w_a null)
//          = coef * (rms(a) * w_a + rms(b) * w_b)   two branches, each divided by its own root mean square (b may be null)
//   z      = y / sqrt(mean(y^2) + eps) * w       the outer norm (w null: z = y)
//   residual += z                                (residual null: z goes to out32)
//   cast   = T(residual)                         (optional: the stream in the activation type, for the next product)
//
// All of it in 32-bit, the row kept in shared memory.  One block per row.
namespace {

template <typename TIN, typename TA, typename TW, int VEC>
__global__ void __launch_bounds__(1024)
branch_norm_kernel(const TIN* __restrict__ a, const TW* __restrict__ wa, const TIN* __restrict__ b,
                   const TW* __restrict__ wb, float coef, float inner_eps, const TW* __restrict__ w, float eps,
                   float* __restrict__ residual, float* __restrict__ out32, TA* __restrict__ cast, int h) {
  extern __shared__ __align__(16) float rows_sm[];        // the row of a, and of b behind it: each is read from memory once
  __shared__ float red[33];
  float* ya = rows_sm;
  float* yb = rows_sm + h;
  pdl_enter();
  const int64_t r = blockIdx.x;
  const TIN* pa = a + r * h;
  const TIN* pb = b ? b + r * h : nullptr;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x * VEC; i < h; i += blockDim.x * VEC) {
    float x[4], y[4];
    if (VEC == 4) { load4<TIN>(pa + i, x); if (pb) load4<TIN>(pb + i, y); }
    else { x[0] = to_f32<TIN>(pa[i]); if (pb) y[0] = to_f32<TIN>(pb[i]); }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      ya[i + j] = x[j];
      sa += x[j] * x[j];
      if (pb) { yb[i + j] = y[j]; sb += y[j] * y[j]; }
    }
  }
  float ss = sa;                                           // one branch without an inner norm: y = a
  if (wa) {
    sa = block_sum(sa, red);
    if (pb) sb = block_sum(sb, red);
    const float ra = 1.f / sqrtf(sa / (float)h + inner_eps);
    const float rb = pb ? 1.f / sqrtf(sb / (float)h + inner_eps) : 0.f;
    ss = 0.f;
    for (int i = threadIdx.x; i < h; i += blockDim.x) {    // behind the barriers of the sums above
      float y = ya[i] * ra * to_f32<TW>(wa[i]);
      if (pb) y += yb[i] * rb * to_f32<TW>(wb[i]);
      y *= coef;
      ya[i] = y;
      ss += y * y;
    }
  }
  float rn = 1.f;
  if (w) rn = 1.f / sqrtf(block_sum(ss, red) / (float)h + eps);
  if (wa && VEC == 4) __syncthreads();                     // the pass above walked the row element by element
  for (int i = threadIdx.x * VEC; i < h; i += blockDim.x * VEC) {
    float z[4], wv[4], res[4];
    if (VEC == 4) {
      if (w) load4<TW>(w + i, wv);
      if (residual) load4<float>(residual + r * h + i, res);
    } else {
      if (w) wv[0] = to_f32<TW>(w[i]);
      if (residual) res[0] = residual[r * h + i];
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
      z[j] = ya[i + j];
      if (w) z[j] = z[j] * rn * wv[j];
      if (residual) z[j] += res[j];
    }
    float* dst = residual ? residual + r * h + i : out32 + r * h + i;
    if (VEC == 4) { store4<float>(dst, z); if (cast) store4<TA>(cast + r * h + i, z); }
    else { dst[0] = z[0]; if (cast) cast[r * h + i] = from_f32<TA>(z[0]); }
  }
}

}  // namespace

// a, b [num_rows, h] of in_dtype (b null: one branch); wa, wb inner weights [h] (wa null: no inner norm); w the outer
// weight [h] (null: none); residual f32 [num_rows, h] updated in place, or null with out32 f32 [num_rows, h];
// cast [num_rows, h] act dtype or null.
DINFER_API int dinfer_branch_norm(const void* a, const void* wa, const void* b, const void* wb, float coef,
                                  float inner_eps, const void* w, float eps, float* residual, float* out32, void* cast,
                                  int num_rows, int h, int in_dtype, int act_dtype, int w_dtype, cudaStream_t stream) {
  if (h <= 0 || num_rows < 0) return refuse(DINFER_BAD_ARGUMENT, "branch_norm: bad sizes rows=%d h=%d", num_rows, h);
  if (!a || (b && (!wa || !wb)) || (!residual && !out32))
    return refuse(DINFER_BAD_ARGUMENT, "branch_norm: a branch without its weight, or no output");
  const size_t row_bytes = (size_t)h * sizeof(float) * (b ? 2 : 1);
  if (row_bytes > 200 * 1024) return refuse(DINFER_BAD_ARGUMENT, "branch_norm: rows of %d above the limit", h);
  if (num_rows == 0) return 0;
  const auto al = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
  const bool vec4 = h % 4 == 0 && al(a) && al(b) && al(w) && al(residual) && al(out32) && al(cast);
  int threads = ((vec4 ? h / 4 : h) + 31) / 32 * 32;
  if (threads > 1024) threads = 1024;
  DINFER_DISPATCH_DTYPE(in_dtype, TIN,
   DINFER_DISPATCH_DTYPE(act_dtype, TA,
    DINFER_DISPATCH_DTYPE(w_dtype, TW, {
      auto k4 = branch_norm_kernel<TIN, TA, TW, 4>;
      auto k1 = branch_norm_kernel<TIN, TA, TW, 1>;
      auto k = vec4 ? k4 : k1;
      if (row_bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)row_bytes);
        if (e != cudaSuccess) return refuse((int)e, "branch_norm: shared memory opt-in failed: %s", cudaGetErrorString(e));
      }
      launch_pdl(k, dim3(num_rows), dim3(threads), row_bytes, stream, (const TIN*)a, (const TW*)wa,
                 (const TIN*)b, (const TW*)wb, coef, inner_eps, (const TW*)w, eps, residual, out32, (TA*)cast, h);
      return cuda_status("branch_norm");
    })));
  return 0;
}
