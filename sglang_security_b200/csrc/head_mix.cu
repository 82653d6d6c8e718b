// Row kernels between an attention kernel and its output projection:
//   head_mix_gate     : for designs that mix the heads' softmax weights with a matrix M [H, H] AFTER the
//                       softmax, w'_h(i, j) = sum_g M[h, g] w_g(i, j), and apply w'_h to the values of
//                       head h's own key/value head c(h).  The mixed output is linear in the weights,
//                           out_h(i) = sum_g M[h, g] * A[c(h)][g](i),   A[c][g](i) = sum_j w_g(i, j) v_c(j),
//                       so the attention kernel produces A (every head's weights on every key/value
//                       head's values, one plane per value head) with its usual online softmax, and this
//                       kernel forms the combination per token, in fp32, and multiplies head h by
//                       sigmoid(gate[t, h]) when a gate is given.
//   sigmoid_gate_mul  : out[t, h * E + e] = x[t, h, e] * sigmoid(g[t, h]) or sigmoid(g[t, h * E + e]),
//                       x given with separate token and head strides so that a head-major product
//                       ([H, T, E]) is gated and laid out token-major in one pass.
#include "common.cuh"

namespace b200 {

constexpr int kMixThreads = 256;

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }

// A thread owns one value column e of one plane c and forms the outputs of that plane's R = H / G heads,
// kMixHeads at a time: the H inputs a[g][e] are loaded once per kMixHeads outputs (coalesced over e),
// the mix row comes from shared memory as a broadcast.
constexpr int kMixHeads = 8;

template <typename TA, typename T>
__global__ void __launch_bounds__(kMixThreads)
head_mix_gate_kernel(const TA* __restrict__ a, int64_t lda, int64_t lda_plane,
                     const float* __restrict__ mix, const T* __restrict__ gate, int64_t ldg,
                     T* __restrict__ out, int64_t ldo, int H, int G, int E) {
  extern __shared__ float mix_s[];                 // [H, H] when it fits, else read through the cache
  const bool in_smem = H * H * sizeof(float) <= 32 * 1024;
  if (in_smem) {
    for (int i = threadIdx.x; i < H * H; i += kMixThreads) mix_s[i] = mix[i];
    __syncthreads();
  }
  const float* m = in_smem ? mix_s : mix;
  const int t = blockIdx.x, R = H / G;
  for (int i = threadIdx.x; i < G * E; i += kMixThreads) {
    const int c = i / E, e = i - c * E;
    const TA* col = a + static_cast<int64_t>(c) * lda_plane + t * lda + e;
    for (int h0 = c * R; h0 < (c + 1) * R; h0 += kMixHeads) {
      const int nh = min(kMixHeads, (c + 1) * R - h0);
      float acc[kMixHeads];
#pragma unroll
      for (int r = 0; r < kMixHeads; ++r) acc[r] = 0.f;
#pragma unroll 8                              // eight loads in flight per thread: the kernel is bound by
      for (int g = 0; g < H; ++g) {                // bytes in flight, not by arithmetic
        const float x = to_float<TA>(col[g * E]);
#pragma unroll
        for (int r = 0; r < kMixHeads; ++r)
          if (r < nh) acc[r] = fmaf(m[(h0 + r) * H + g], x, acc[r]);
      }
#pragma unroll
      for (int r = 0; r < kMixHeads; ++r) {
        if (r < nh) {
          float o = acc[r];
          if (gate) o *= sigmoidf_(to_float<T>(gate[t * ldg + h0 + r]));
          out[t * ldo + (h0 + r) * E + e] = from_float<T>(o);
        }
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(kMixThreads)
sigmoid_gate_mul_kernel(const T* __restrict__ x, int64_t ldx_t, int64_t ldx_h, const T* __restrict__ g,
                        int64_t ldg, int per_head, T* __restrict__ out, int64_t ldo, int H, int E) {
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H * E; i += kMixThreads) {
    const int h = i / E, e = i - h * E;
    const float z = to_float<T>(g[t * ldg + (per_head ? h : i)]);
    out[t * ldo + i] = from_float<T>(to_float<T>(x[t * ldx_t + h * ldx_h + e]) * sigmoidf_(z));
  }
}

}  // namespace b200

// a: [G planes of lda_plane][T rows of lda][H, E] (a_dtype: the activations' type, or fp32);
// mix fp32 [H, H] row-major; gate [T rows of ldg][H] or NULL; out [T rows of ldo][H * E].
extern "C" int b200_head_mix_gate(const void* a, int64_t lda, int64_t lda_plane, int a_dtype,
                                  const float* mix, const void* gate, int64_t ldg, void* out,
                                  int64_t ldo, int T, int H, int G, int E, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(a && mix && out && T > 0 && H > 0 && G > 0 && H % G == 0 && E > 0,
               "b200_head_mix_gate: bad arguments (heads %d / %d, value size %d)", H, G, E);
  B200_REQUIRE(a_dtype == dtype || a_dtype == B200_F32, "b200_head_mix_gate: a_dtype %d", a_dtype);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("head_mix_gate", st);
  const size_t smem = static_cast<size_t>(H) * H * 4 <= 32 * 1024 ? static_cast<size_t>(H) * H * 4 : 0;
#define LAUNCH(TA, TT)                                                                               \
  launch_kernel(head_mix_gate_kernel<TA, TT>, dim3(T), dim3(kMixThreads), smem, st, 1, 0,            \
                static_cast<const TA*>(a), lda, lda_plane, mix, static_cast<const TT*>(gate), ldg,   \
                static_cast<TT*>(out), ldo, H, G, E)
  if (dtype == B200_BF16) {
    if (a_dtype == B200_F32) LAUNCH(float, __nv_bfloat16);
    else LAUNCH(__nv_bfloat16, __nv_bfloat16);
  } else if (dtype == B200_F16) {
    if (a_dtype == B200_F32) LAUNCH(float, __half);
    else LAUNCH(__half, __half);
  } else if (dtype == B200_F32) {
    LAUNCH(float, float);
  } else {
    B200_REQUIRE(false, "b200_head_mix_gate: dtype %d", dtype);
  }
#undef LAUNCH
  B200_CHECK_LAUNCH("head_mix_gate_kernel");
  return 0;
}

extern "C" int b200_sigmoid_gate_mul(const void* x, int64_t ldx_t, int64_t ldx_h, const void* g,
                                     int64_t ldg, int per_head, void* out, int64_t ldo, int T, int H,
                                     int E, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(x && g && out && T > 0 && H > 0 && E > 0, "b200_sigmoid_gate_mul: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("sigmoid_gate_mul", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(sigmoid_gate_mul_kernel<TT>, dim3(T), dim3(kMixThreads), 0, st, 1, 0,                \
                static_cast<const TT*>(x), ldx_t, ldx_h, static_cast<const TT*>(g), ldg, per_head,   \
                static_cast<TT*>(out), ldo, H, E)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_sigmoid_gate_mul: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("sigmoid_gate_mul_kernel");
  return 0;
}
