// Row kernels around a 32-bit residual stream, for model designs that keep the residual, the norms
// and the previous-token mix in fp32 while the matrix products run in the model dtype:
//   scalar_rmsnorm_shift : h = x / sqrt(mean(x^2) + eps) * gain (* weight[d]), and optionally the
//                          token-shifted copy hm = h + (h_prev - h) * mu[d], where h_prev is the h of
//                          the previous token of the same sequence: the row before it in this batch,
//                          the per-sequence state row if the token opens its portion, zeros at
//                          position 0.  The state row is replaced by the h of the portion's last token.
//   residual_combine     : x += a + b + sum_k w[t,k] * y[t*top+k] + g[t] * s[t]   (all terms optional)
//   act_and_mul          : out = act(z[:, :d]) * z[:, d:]  with act = silu or the tanh form of gelu
//   add_normed           : for designs whose norm sits on a sublayer's OUTPUT: y = sa * a + sb * b +
//                          sum_k rows[t * top + k] (all terms optional) in fp32, then
//                          x += mult * y / sqrt(mean(y^2) + eps) * w[d]; optionally also writes the new x
//                          in the model dtype, the next sublayer's input; with a second weight the copy is
//                          the NEXT sublayer's pre-norm instead, x / sqrt(mean(x^2) + eps) * w_next (designs
//                          with a norm on both sides of every sublayer: one launch per sublayer boundary)
//   softcap_rows         : out = cap * tanh(z / cap) in fp32
//   scaled_add_layernorm : for designs whose norm sits AFTER the residual sum: y = alpha * x + a + b +
//                          sum_k wts[t, k] * rows[t * top + k] (terms optional) in fp32, then
//                          x = (y - mean) / sqrt(var + eps) * w + bias (two passes: the variance is the
//                          mean of the squared deviations); optionally the copy of the new x in the
//                          model dtype.  With `in_place` = 0 x is left alone and only the copy is
//                          written (a model's final layer norm).
//   act_and_mul_clamped  : out = g * sigmoid(slope * g) * (u + 1), g = min(z[:, :d], limit),
//                          u = clamp(z[:, d:], -limit, limit)
#include "common.cuh"

namespace b200 {

constexpr int kRowThreads = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();  // red may still be read from the previous call
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < kRowThreads / 32) ? red[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

__device__ __forceinline__ float row_inv_rms(const float* row, int W, float eps, float* red) {
  float s = 0.f;
  for (int d = threadIdx.x; d < W; d += kRowThreads) {
    const float v = row[d];
    s = fmaf(v, v, s);
  }
  s = block_sum(s, red);
  return 1.0f / sqrtf(s / static_cast<float>(W) + eps);
}

template <typename TO>
__global__ void __launch_bounds__(kRowThreads)
scalar_rmsnorm_shift_kernel(const float* __restrict__ x, int64_t ldx, const float* __restrict__ gain,
                            const float* __restrict__ weight, float eps,
                            const float* __restrict__ mu, float* __restrict__ state, int64_t ld_state,
                            const int* __restrict__ tok_pos, const int* __restrict__ tok_b,
                            const int* __restrict__ ext_start, const int* __restrict__ ext_len,
                            const int64_t* __restrict__ slot, TO* __restrict__ out_h, int64_t ldh,
                            TO* __restrict__ out_hm, int64_t ldm, int W) {
  __shared__ float red[kRowThreads / 32];
  const int t = blockIdx.x;
  const float g = gain ? *gain : 1.0f;
  const float* row = x + t * ldx;
  const float r = row_inv_rms(row, W, eps, red) ;
  if (!mu) {
    for (int d = threadIdx.x; d < W; d += kRowThreads) {
      float h = row[d] * r * g;
      if (weight) h *= weight[d];
      out_h[t * ldh + d] = from_float<TO>(h);
    }
    return;
  }
  const int b = tok_b[t];
  const int start = ext_start[b];
  const bool first = (t == start);
  const int pos = tok_pos[t];
  // 0: zeros, 1: the state row, 2: the previous row of this batch
  const int src = pos == 0 ? 0 : (first ? 1 : 2);
  float rp = 0.f;
  const float* prow = row - ldx;
  if (src == 2) rp = row_inv_rms(prow, W, eps, red);
  const int last = start + ext_len[b] - 1;
  float* srow = state ? state + slot[b] * ld_state : nullptr;
  float rl = r;
  const float* lrow = x + last * ldx;
  if (first && srow && last != t) rl = row_inv_rms(lrow, W, eps, red);
  for (int d = threadIdx.x; d < W; d += kRowThreads) {
    const float wd = weight ? weight[d] * g : g;
    const float h = row[d] * r * wd;
    float hp = 0.f;
    if (src == 1) hp = srow[d];
    else if (src == 2) hp = prow[d] * rp * wd;
    if (out_h) out_h[t * ldh + d] = from_float<TO>(h);
    out_hm[t * ldm + d] = from_float<TO>(h + (hp - h) * mu[d]);
    if (first && srow) srow[d] = (last == t) ? h : lrow[d] * rl * wd;   // same thread read srow[d] above
  }
}

template <typename TA>
__global__ void __launch_bounds__(kRowThreads)
residual_combine_kernel(float* __restrict__ x, int64_t ldx, const TA* __restrict__ a, int64_t lda,
                        const TA* __restrict__ b, int64_t ldb, const TA* __restrict__ y, int64_t ldy,
                        const float* __restrict__ topk_w, int top, const TA* __restrict__ s,
                        int64_t lds, const float* __restrict__ gate, int W) {
  const int t = blockIdx.x;
  const float g = gate ? gate[t] : 1.0f;
  for (int d = threadIdx.x; d < W; d += kRowThreads) {
    float acc = 0.f;
    if (a) acc += to_float<TA>(a[t * lda + d]);
    if (b) acc += to_float<TA>(b[t * ldb + d]);
    if (y) {
      float m = 0.f;
      for (int k = 0; k < top; ++k)
        m = fmaf(topk_w[t * top + k], to_float<TA>(y[(static_cast<int64_t>(t) * top + k) * ldy + d]), m);
      acc += m;
    }
    if (s) acc = fmaf(g, to_float<TA>(s[t * lds + d]), acc);
    x[t * ldx + d] += acc;
  }
}

__device__ __forceinline__ float act_apply(float z, int kind) {
  if (kind == 0) return z / (1.0f + expf(-z));                      // silu
  const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);  // gelu, tanh form
  return 0.5f * z * (1.0f + tanhf(u));
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
act_and_mul_kernel(const T* __restrict__ z, int64_t ldz, T* __restrict__ out, int64_t ldo, int D,
                   int kind) {
  const int t = blockIdx.x;
  for (int d = threadIdx.x; d < D; d += kRowThreads) {
    // the activation's value is rounded to the storage type before the product, as a chain of
    // separate operators would round it
    const float a = to_float<T>(from_float<T>(act_apply(to_float<T>(z[t * ldz + d]), kind)));
    out[t * ldo + d] = from_float<T>(a * to_float<T>(z[t * ldz + D + d]));
  }
}

template <typename TA>
__global__ void __launch_bounds__(kRowThreads)
add_normed_kernel(float* __restrict__ x, int64_t ldx, const TA* __restrict__ a, int64_t lda, float sa,
                  const TA* __restrict__ b, int64_t ldb, float sb, const TA* __restrict__ y,
                  int64_t ldy, int top, const float* __restrict__ w, float eps, float mult,
                  TA* __restrict__ out_h, int64_t ldh, int W, const float* __restrict__ w_next) {
  __shared__ float red[kRowThreads / 32];
  const int t = blockIdx.x;
  auto term = [&](int d) {
    float v = 0.f;
    if (a) v = sa * to_float<TA>(a[t * lda + d]);
    if (b) v = fmaf(sb, to_float<TA>(b[t * ldb + d]), v);
    if (y)
      for (int k = 0; k < top; ++k) v += to_float<TA>(y[(static_cast<int64_t>(t) * top + k) * ldy + d]);
    return v;
  };
  float s = 0.f;
  for (int d = threadIdx.x; d < W; d += kRowThreads) {
    const float v = term(d);
    s = fmaf(v, v, s);
  }
  s = block_sum(s, red);
  const float r = mult / sqrtf(s / static_cast<float>(W) + eps);
  float s2 = 0.f;
  for (int d = threadIdx.x; d < W; d += kRowThreads) {
    const float nx = fmaf(term(d) * r, w ? w[d] : 1.f, x[t * ldx + d]);
    x[t * ldx + d] = nx;
    s2 = fmaf(nx, nx, s2);
    if (out_h && !w_next) out_h[t * ldh + d] = from_float<TA>(nx);
  }
  if (!out_h || !w_next) return;
  // the next sublayer's pre-norm of the new residual (each thread re-reads the elements it wrote)
  s2 = block_sum(s2, red);
  const float r2 = 1.0f / sqrtf(s2 / static_cast<float>(W) + eps);
  for (int d = threadIdx.x; d < W; d += kRowThreads)
    out_h[t * ldh + d] = from_float<TA>(x[t * ldx + d] * r2 * w_next[d]);
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
softcap_rows_kernel(const T* __restrict__ z, int64_t ldz, float* __restrict__ out, int64_t ldo, int V,
                    float cap) {
  const int t = blockIdx.x;
  for (int d = threadIdx.x; d < V; d += kRowThreads) {
    const float v = to_float<T>(z[t * ldz + d]);
    out[t * ldo + d] = cap > 0.f ? cap * tanhf(v / cap) : v;
  }
}

template <typename TA, typename TO>
__global__ void __launch_bounds__(kRowThreads)
scaled_add_layernorm_kernel(float* __restrict__ x, int64_t ldx, float alpha, const TA* __restrict__ a,
                            int64_t lda, const TA* __restrict__ b, int64_t ldb,
                            const TA* __restrict__ rows, int64_t ld_rows,
                            const float* __restrict__ wts, int top, const float* __restrict__ w,
                            const float* __restrict__ bias, float eps, TO* __restrict__ out_h,
                            int64_t ldh, int W, int in_place) {
  extern __shared__ float ln_row[];          // [W] the summed row
  __shared__ float red[kRowThreads / 32];
  const int t = blockIdx.x;
  float s = 0.f;
  for (int d = threadIdx.x; d < W; d += kRowThreads) {
    float v = alpha * x[t * ldx + d];
    if (a) v += to_float<TA>(a[t * lda + d]);
    if (rows)
      for (int k = 0; k < top; ++k)
        v = fmaf(wts ? wts[t * top + k] : 1.f, to_float<TA>(rows[(static_cast<int64_t>(t) * top + k) * ld_rows + d]), v);
    if (b) v += to_float<TA>(b[t * ldb + d]);
    ln_row[d] = v;
    s += v;
  }
  const float mean = block_sum(s, red) / static_cast<float>(W);
  float q = 0.f;
  for (int d = threadIdx.x; d < W; d += kRowThreads) {
    const float c = ln_row[d] - mean;
    q = fmaf(c, c, q);
  }
  const float r = 1.0f / sqrtf(block_sum(q, red) / static_cast<float>(W) + eps);
  for (int d = threadIdx.x; d < W; d += kRowThreads) {
    const float y = fmaf((ln_row[d] - mean) * r, w ? w[d] : 1.f, bias ? bias[d] : 0.f);
    if (in_place) x[t * ldx + d] = y;
    if (out_h) out_h[t * ldh + d] = from_float<TO>(y);
  }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads)
act_and_mul_clamped_kernel(const T* __restrict__ z, int64_t ldz, T* __restrict__ out, int64_t ldo, int D,
                           float limit, float slope) {
  const int t = blockIdx.x;
  for (int d = threadIdx.x; d < D; d += kRowThreads) {
    const float g = fminf(to_float<T>(z[t * ldz + d]), limit);
    const float u = fminf(fmaxf(to_float<T>(z[t * ldz + D + d]), -limit), limit);
    out[t * ldo + d] = from_float<T>(g / (1.0f + expf(-slope * g)) * (u + 1.0f));
  }
}

}  // namespace b200

extern "C" int b200_scalar_rmsnorm_shift(const float* x, int64_t ldx, const float* gain,
                                         const float* weight, float eps, const float* mu,
                                         float* state, int64_t ld_state, const int* tok_pos,
                                         const int* tok_b, const int* ext_start, const int* ext_len,
                                         const int64_t* slot, void* out_h, int64_t ldh, void* out_hm,
                                         int64_t ldm, int T, int W, int out_dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(x && (out_h || out_hm) && T > 0 && W > 0, "b200_scalar_rmsnorm_shift: bad arguments");
  B200_REQUIRE(!mu || (out_hm && tok_pos && tok_b && ext_start && ext_len),
               "b200_scalar_rmsnorm_shift: the shift needs out_hm and the token/portion tables");
  B200_REQUIRE(mu || out_h, "b200_scalar_rmsnorm_shift: out_h is NULL");
  B200_REQUIRE(!state || slot, "b200_scalar_rmsnorm_shift: state without slots");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("scalar_rmsnorm_shift", st);
#define LAUNCH(TO)                                                                                   \
  launch_kernel(scalar_rmsnorm_shift_kernel<TO>, dim3(T), dim3(kRowThreads), 0, st, 1, 0, x, ldx,   \
                gain, weight, eps, mu, state, ld_state, tok_pos, tok_b, ext_start, ext_len, slot,    \
                static_cast<TO*>(out_h), ldh, static_cast<TO*>(out_hm), ldm, W)
  if (out_dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (out_dtype == B200_F16) LAUNCH(__half);
  else if (out_dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_scalar_rmsnorm_shift: dtype %d", out_dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("scalar_rmsnorm_shift_kernel");
  return 0;
}

extern "C" int b200_residual_combine(float* x, int64_t ldx, const void* a, int64_t lda, const void* b,
                                     int64_t ldb, const void* y, int64_t ldy, const float* topk_w,
                                     int top, const void* s, int64_t lds, const float* gate, int T,
                                     int W, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(x && T > 0 && W > 0, "b200_residual_combine: bad arguments");
  B200_REQUIRE(!y || (topk_w && top > 0), "b200_residual_combine: expert rows without weights");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("residual_combine", st);
#define LAUNCH(TA)                                                                                   \
  launch_kernel(residual_combine_kernel<TA>, dim3(T), dim3(kRowThreads), 0, st, 1, 0, x, ldx,       \
                static_cast<const TA*>(a), lda, static_cast<const TA*>(b), ldb,                      \
                static_cast<const TA*>(y), ldy, topk_w, top, static_cast<const TA*>(s), lds, gate, W)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_residual_combine: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("residual_combine_kernel");
  return 0;
}

extern "C" int b200_act_and_mul(const void* z, int64_t ldz, void* out, int64_t ldo, int T, int D,
                                int kind, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(z && out && T > 0 && D > 0 && (kind == 0 || kind == 1), "b200_act_and_mul: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("act_and_mul", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(act_and_mul_kernel<TT>, dim3(T), dim3(kRowThreads), 0, st, 1, 0,                    \
                static_cast<const TT*>(z), ldz, static_cast<TT*>(out), ldo, D, kind)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_act_and_mul: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("act_and_mul_kernel");
  return 0;
}

extern "C" int b200_add_normed_next(float* x, int64_t ldx, const void* a, int64_t lda, float sa,
                                    const void* b, int64_t ldb, float sb, const void* rows,
                                    int64_t ld_rows, int top, const float* w, float eps, float mult,
                                    void* out_h, int64_t ldh, const float* w_next, int T, int W,
                                    int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(x && (a || b || rows) && T > 0 && W > 0, "b200_add_normed: bad arguments");
  B200_REQUIRE(!rows || top > 0, "b200_add_normed: rows without a count per token");
  B200_REQUIRE(!w_next || out_h, "b200_add_normed: a next norm without an output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("add_normed", st);
#define LAUNCH(TA)                                                                                   \
  launch_kernel(add_normed_kernel<TA>, dim3(T), dim3(kRowThreads), 0, st, 1, 0, x, ldx,             \
                static_cast<const TA*>(a), lda, sa, static_cast<const TA*>(b), ldb, sb,              \
                static_cast<const TA*>(rows), ld_rows, top, w, eps, mult, static_cast<TA*>(out_h),   \
                ldh, W, w_next)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_add_normed: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("add_normed_kernel");
  return 0;
}

extern "C" int b200_add_normed(float* x, int64_t ldx, const void* a, int64_t lda, float sa,
                               const void* b, int64_t ldb, float sb, const void* rows, int64_t ld_rows,
                               int top, const float* w, float eps, float mult, void* out_h, int64_t ldh,
                               int T, int W, int dtype, void* stream) {
  return b200_add_normed_next(x, ldx, a, lda, sa, b, ldb, sb, rows, ld_rows, top, w, eps, mult, out_h,
                              ldh, nullptr, T, W, dtype, stream);
}

extern "C" int b200_softcap_rows(const void* z, int64_t ldz, float* out, int64_t ldo, int T, int V,
                                 float cap, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(z && out && T > 0 && V > 0, "b200_softcap_rows: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("softcap_rows", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(softcap_rows_kernel<TT>, dim3(T), dim3(kRowThreads), 0, st, 1, 0,                   \
                static_cast<const TT*>(z), ldz, out, ldo, V, cap)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_softcap_rows: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("softcap_rows_kernel");
  return 0;
}

extern "C" int b200_scaled_add_layernorm(float* x, int64_t ldx, float alpha, const void* a, int64_t lda,
                                         const void* b, int64_t ldb, const void* rows, int64_t ld_rows,
                                         const float* wts, int top, const float* w, const float* bias,
                                         float eps, void* out_h, int64_t ldh, int in_place, int T, int W,
                                         int dtype, int out_dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(x && T > 0 && W > 0 && (in_place || out_h), "b200_scaled_add_layernorm: bad arguments");
  B200_REQUIRE(!rows || top > 0, "b200_scaled_add_layernorm: rows without a count per token");
  B200_REQUIRE(out_dtype == dtype || out_dtype == B200_F32 || !out_h,
               "b200_scaled_add_layernorm: the copy has the terms' dtype or fp32");
  const size_t smem = sizeof(float) * static_cast<size_t>(W);
  B200_REQUIRE(smem <= 200 * 1024, "b200_scaled_add_layernorm: width %d too large", W);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("scaled_add_layernorm", st);
#define LAUNCH(TA, TO)                                                                               \
  do {                                                                                               \
    if (smem > 48 * 1024)                                                                            \
      B200_CUDA_OK(cudaFuncSetAttribute(scaled_add_layernorm_kernel<TA, TO>,                         \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
    launch_kernel(scaled_add_layernorm_kernel<TA, TO>, dim3(T), dim3(kRowThreads), smem, st, 1, 0, x, \
                  ldx, alpha, static_cast<const TA*>(a), lda, static_cast<const TA*>(b), ldb,        \
                  static_cast<const TA*>(rows), ld_rows, wts, top, w, bias, eps,                     \
                  static_cast<TO*>(out_h), ldh, W, in_place);                                        \
  } while (0)
  if (dtype == B200_BF16 && out_dtype == B200_F32) LAUNCH(__nv_bfloat16, float);
  else if (dtype == B200_F16 && out_dtype == B200_F32) LAUNCH(__half, float);
  else if (dtype == B200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half, __half);
  else if (dtype == B200_F32) LAUNCH(float, float);
  else B200_REQUIRE(false, "b200_scaled_add_layernorm: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("scaled_add_layernorm_kernel");
  return 0;
}

extern "C" int b200_act_and_mul_clamped(const void* z, int64_t ldz, void* out, int64_t ldo, int T, int D,
                                        float limit, float slope, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(z && out && T > 0 && D > 0 && limit > 0.f, "b200_act_and_mul_clamped: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("act_and_mul_clamped", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(act_and_mul_clamped_kernel<TT>, dim3(T), dim3(kRowThreads), 0, st, 1, 0,            \
                static_cast<const TT*>(z), ldz, static_cast<TT*>(out), ldo, D, limit, slope)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_act_and_mul_clamped: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("act_and_mul_clamped_kernel");
  return 0;
}
