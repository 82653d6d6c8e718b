// Recurrent mixers whose memory is a matrix S [D key rows, E value columns] per head, kept in fp32 and
// carried from token to token, with a decay that is computed from the token (not a constant), and the
// short causal convolution that feeds them.
//
//   causal_conv_silu  : y[t, c] = silu(bias[c] + sum_j w[c, taps-1-j] * x[t-j, c]) over the tokens of a
//                       sequence; x before position 0 is zero.  The inputs of a portion's first tokens
//                       that lie before the portion come from the sequence's state row, which holds the
//                       last taps-1 inputs ([taps-1, C] fp32, oldest first).
//   conv_state_update : after the convolution has read it, the state row takes the last taps-1 inputs
//                       of the portion (shifting what it held when the portion is shorter).
//   delta_recurrence  : per (sequence, head), token by token
//                         mode 0 (delta rule, a decay per key row):
//                           g_r = exp(-exp(A_h) * softplus(raw[t, h, r] + bias[h, r]))
//                           S <- diag(g) S ; u = beta (v - S^T k) ; S <- S + k u^T ; o = S^T q
//                           with q, k divided by sqrt(sum(x^2) + unit_eps), q times q_scale, beta =
//                           sigmoid(beta_raw[t, h])
//                         mode 1 (state space, a scalar decay per head):
//                           dt = softplus(raw[t, h] + bias[h]) ; a = exp(-exp(A_h) dt)
//                           S <- a S + k (dt v)^T ; o = S^T q + skip_h v
//                       Two launches.  What does not depend on the memory (unit vectors, decays, write
//                       strengths, step sizes) is prepared for all tokens of the step in parallel, one
//                       CTA per token, as fp32 rows of a workspace.  The scan then walks each (sequence,
//                       head) in order: a thread owns RPL rows of one value column of S in registers (LPC
//                       lanes share a column and reduce by shuffles), so a token costs two passes over
//                       the thread's rows and no shared-memory traffic for S; the prepared rows of the
//                       next 16 tokens stream into the other half of a double buffer (cp.async) while
//                       the current ones are walked.  Every sum is taken in an order that depends on
//                       neither the chunking, the portion nor the CTA shape, so prefill, portions and
//                       single decoded tokens give identical results.  State row layout: [H][D][E] fp32;
//                       a portion that starts at position 0 ignores what the row holds.
#include "common.cuh"

namespace b200 {

constexpr int kConvThreads = 256;

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
causal_conv_silu_kernel(const T* __restrict__ x, int64_t ldx, const float* __restrict__ w,
                        const float* __restrict__ bias, const float* __restrict__ state,
                        int64_t ld_state, const int64_t* __restrict__ slot,
                        const int* __restrict__ tok_pos, const int* __restrict__ tok_b,
                        const int* __restrict__ ext_start, T* __restrict__ out, int64_t ldo, int C,
                        int taps) {
  const int t = blockIdx.x, c = blockIdx.y * kConvThreads + threadIdx.x;
  if (c >= C) return;
  const int b = tok_b[t], i = t - ext_start[b], p = tok_pos[t];
  const float* st = state + slot[b] * ld_state;
  float acc = bias ? bias[c] : 0.f;
  for (int j = 0; j < taps && j <= p; ++j) {       // j tokens back; before position 0: zeros
    const float xin = j <= i ? to_float<T>(x[static_cast<int64_t>(t - j) * ldx + c])
                             : st[static_cast<int64_t>(taps - 1 - (j - i)) * C + c];
    acc = fmaf(w[c * taps + taps - 1 - j], xin, acc);
  }
  out[t * ldo + c] = from_float<T>(acc / (1.0f + expf(-acc)));
}

template <typename T>
__global__ void __launch_bounds__(kConvThreads)
conv_state_update_kernel(const T* __restrict__ x, int64_t ldx, float* __restrict__ state,
                         int64_t ld_state, const int64_t* __restrict__ slot,
                         const int* __restrict__ tok_pos, const int* __restrict__ ext_start,
                         const int* __restrict__ ext_len, int C, int taps) {
  const int b = blockIdx.x, c = blockIdx.y * kConvThreads + threadIdx.x;
  const int n = ext_len[b];
  if (c >= C || n <= 0) return;
  const int r0 = ext_start[b], p0 = tok_pos[r0];
  float* st = state + slot[b] * ld_state;
  for (int s = 0; s < taps - 1; ++s) {             // increasing s: what is read lies ahead of what is written
    const int idx = n - (taps - 1) + s;            // the input to keep, relative to the portion's start
    float v = 0.f;
    if (idx >= 0) v = to_float<T>(x[static_cast<int64_t>(r0 + idx) * ldx + c]);
    else if (p0 + idx >= 0) v = st[static_cast<int64_t>(s + n) * C + c];
    st[static_cast<int64_t>(s) * C + c] = v;
  }
}

constexpr int kDeltaChunk = 16;   // tokens staged at a time (fewer when the rows are very long)

// Per token, everything of the recurrence that does not depend on the memory, in parallel over all
// tokens of the step (one CTA per token), as fp32 rows of a workspace:
//   kq [T, 2 * G * D]  keys, then queries (delta rule: unit vectors, the query times q_scale)
//   g  [T, H * D]      decay per key row (delta rule only)
//   ab [T, 2 * H]      write strength beta (delta rule) or step size dt, then the scalar decay
template <typename T, bool DELTA>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                     const T* __restrict__ decay_raw, int64_t ld_decay,
                     const float* __restrict__ decay_bias, const float* __restrict__ a_log,
                     const T* __restrict__ beta_raw, int64_t ld_beta, float q_scale, float unit_eps,
                     float* __restrict__ kq, float* __restrict__ g, float* __restrict__ ab, int H, int G,
                     int D) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* kq_t = kq + static_cast<int64_t>(t) * 2 * G * D;
  // one warp per (keys | queries, group): lanes stride over the rows, a fixed shuffle tree
  for (int job = warp; job < 2 * G; job += 8) {
    const bool is_q = job >= G;
    const int c = is_q ? job - G : job;
    const T* src = (is_q ? q + t * ldq : k + t * ldk) + c * D;
    float* dst = kq_t + job * D;
    float scale = 1.f;
    if (DELTA) {
      float ss = 0.f;
      for (int r = lane; r < D; r += 32) {
        const float x = to_float<T>(src[r]);
        ss = fmaf(x, x, ss);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      scale = (is_q ? q_scale : 1.0f) / sqrtf(ss + unit_eps);
    }
    for (int r = lane; r < D; r += 32) dst[r] = to_float<T>(src[r]) * scale;
  }
  if (DELTA) {
    for (int i = threadIdx.x; i < H * D; i += 256)
      g[static_cast<int64_t>(t) * H * D + i] =
          expf(-expf(a_log[i / D]) * softplus_f(to_float<T>(decay_raw[t * ld_decay + i]) + decay_bias[i]));
  }
  for (int h = threadIdx.x; h < H; h += 256) {
    float bv, av = 1.f;
    if (DELTA) {
      bv = 1.0f / (1.0f + expf(-to_float<T>(beta_raw[t * ld_beta + h])));
    } else {
      bv = softplus_f(to_float<T>(decay_raw[t * ld_decay + h]) + decay_bias[h]);
      av = expf(-expf(a_log[h]) * bv);
    }
    ab[static_cast<int64_t>(t) * 2 * H + h] = bv;
    ab[static_cast<int64_t>(t) * 2 * H + H + h] = av;
  }
}

struct DeltaArgs {
  const void* v;
  int64_t ldv;
  const float *kq, *g, *ab;      // prepared rows (delta_prepare_kernel)
  const float* skip;
  float* state;
  int64_t ld_state;
  const int64_t* slot;
  const int *tok_pos, *ext_start, *ext_len;
  float* out;
  int64_t ldo;
  int H, G, D, E, lpc, chunk;
};

__device__ __forceinline__ void cp_async4(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(smem_addr), "l"(gptr));
}

// The scan: S stays in registers, the prepared rows of the next chunk of tokens stream into the other
// half of a double buffer (cp.async) while the current chunk is walked.
template <typename T, int RPL, bool DELTA>
__global__ void __launch_bounds__(128)
delta_recurrence_kernel(const DeltaArgs a) {
  extern __shared__ __align__(16) float dr_smem[];
  const int b = blockIdx.x, h = blockIdx.y, LPC = a.lpc, Dp = RPL * LPC, CH = a.chunk;
  const int D = a.D, E = a.E, H = a.H, G = a.G, c = h / (H / G);
  const int n = a.ext_len[b];
  if (n <= 0) return;
  const int row0 = a.ext_start[b], pos0 = a.tok_pos[row0];
  const int tid = threadIdx.x, nt = blockDim.x;
  const int cols = nt / LPC, part = tid % LPC;
  const int e = blockIdx.z * cols + tid / LPC;
  const bool live = e < E;
  // one buffer: ks [CH][Dp], qs [CH][Dp], gs [CH][Dp] (delta), bs [CH], as [CH], vs [CH][cols]
  const int buf_floats = (CH * Dp * (DELTA ? 3 : 2) + 2 * CH + CH * cols + 3) & ~3;   // halves stay 16-byte aligned
  const T* vg = static_cast<const T*>(a.v);
  const float skip = (!DELTA && a.skip) ? a.skip[h] : 0.f;
  float* srow = a.state + a.slot[b] * a.ld_state + static_cast<int64_t>(h) * D * E;
  // rows past D stay zero (keys, queries) and one (decays) in both buffers: only rows < D are staged
  for (int i = tid; i < 2 * buf_floats; i += nt) dr_smem[i] = 0.f;
  __syncthreads();
  const bool vec4 = (D % 4 == 0);              // the workspace rows then start on 16-byte boundaries
  // how this CTA's slice of a value row can be copied: every piece must start on a multiple of its size
  // in global and in shared memory and the slice must be whole pieces
  int v_mode = 0;
  {
    const int c0 = blockIdx.z * cols, nc = min(cols, E - c0);
    const uintptr_t first = reinterpret_cast<uintptr_t>(vg + h * E + c0);
    const size_t row_bytes = static_cast<size_t>(a.ldv) * sizeof(T), slice = nc * sizeof(T),
                 srow_bytes = cols * sizeof(T);
    if (first % 16 == 0 && row_bytes % 16 == 0 && slice % 16 == 0 && srow_bytes % 16 == 0 && CH % 2 == 0) v_mode = 16;
    else if (first % 4 == 0 && row_bytes % 4 == 0 && slice % 4 == 0 && srow_bytes % 4 == 0) v_mode = 4;
  }

  auto stage = [&](int t0, float* buf) {
    const int m = min(CH, n - t0);
    float* ks = buf;
    float* qs = ks + CH * Dp;
    float* gs = qs + CH * Dp;
    float* bs = buf + CH * Dp * (DELTA ? 3 : 2);
    float* as = bs + CH;
    float* vs = as + CH;
    const int per = vec4 ? D / 4 : D;
    for (int idx = tid; idx < m * per; idx += nt) {
      const int tt = idx / per, r = (idx - tt * per) * (vec4 ? 4 : 1);
      const int64_t row = row0 + t0 + tt;
      const float* ksrc = a.kq + row * 2 * G * D + c * D + r;
      const float* qsrc = a.kq + row * 2 * G * D + (G + c) * D + r;
      if (vec4) {
        cp_async16(smem_u32(ks + tt * Dp + r), ksrc);
        cp_async16(smem_u32(qs + tt * Dp + r), qsrc);
        if (DELTA) cp_async16(smem_u32(gs + tt * Dp + r), a.g + row * H * D + h * D + r);
      } else {
        cp_async4(smem_u32(ks + tt * Dp + r), ksrc);
        cp_async4(smem_u32(qs + tt * Dp + r), qsrc);
        if (DELTA) cp_async4(smem_u32(gs + tt * Dp + r), a.g + row * H * D + h * D + r);
      }
    }
    for (int tt = tid; tt < m; tt += nt) {
      const int64_t row = row0 + t0 + tt;
      cp_async4(smem_u32(bs + tt), a.ab + row * 2 * H + h);
      cp_async4(smem_u32(as + tt), a.ab + row * 2 * H + H + h);
    }
    // values stay in their own type (converted where they are used): 16-byte or 4-byte asynchronous copies
    // when the slice of the row allows it, plain loads otherwise
    T* vraw = reinterpret_cast<T*>(vs);
    const int c0 = blockIdx.z * cols, nc = min(cols, E - c0);
    if (v_mode == 16 || v_mode == 4) {
      const int per_v = static_cast<int>(v_mode / sizeof(T)), pieces = nc / per_v;
      for (int idx = tid; idx < m * pieces; idx += nt) {
        const int tt = idx / pieces, cl = (idx - tt * pieces) * per_v;
        const T* src = vg + (row0 + t0 + tt) * a.ldv + h * E + c0 + cl;
        if (v_mode == 16) cp_async16(smem_u32(vraw + tt * cols + cl), src);
        else cp_async4(smem_u32(vraw + tt * cols + cl), src);
      }
    } else {
      for (int idx = tid; idx < m * nc; idx += nt) {
        const int tt = idx / nc, cl = idx - tt * nc;
        vraw[tt * cols + cl] = vg[(row0 + t0 + tt) * a.ldv + h * E + c0 + cl];
      }
    }
    cp_async_commit();
  };

  float S[RPL];
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = i * LPC + part;
    S[i] = (pos0 > 0 && live && r < D) ? srow[static_cast<int64_t>(r) * E + e] : 0.f;
  }
  stage(0, dr_smem);
  int cur = 0;
  for (int t0 = 0; t0 < n; t0 += CH, cur ^= 1) {
    const int m = min(CH, n - t0);
    float* buf = dr_smem + cur * buf_floats;
    if (t0 + CH < n) {
      stage(t0 + CH, dr_smem + (cur ^ 1) * buf_floats);   // the other half was released by the barrier below
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const float* ks = buf;
    const float* qs = ks + CH * Dp;
    const float* gs = qs + CH * Dp;
    const float* bs = buf + CH * Dp * (DELTA ? 3 : 2);
    const float* as = bs + CH;
    const T* vs = reinterpret_cast<const T*>(as + CH);
#pragma unroll 1
    for (int tt = 0; tt < m; ++tt) {
      const float vt = live ? to_float<T>(vs[tt * cols + tid / LPC]) : 0.f;
      const float* kt = ks + tt * Dp + part;
      const float* qt = qs + tt * Dp + part;
      float u;
      if (DELTA) {
        const float* gt = gs + tt * Dp + part;
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
        for (int i = 0; i < RPL; i += 4) {
          S[i] *= gt[i * LPC];
          S[i + 1] *= gt[(i + 1) * LPC];
          S[i + 2] *= gt[(i + 2) * LPC];
          S[i + 3] *= gt[(i + 3) * LPC];
          d0 = fmaf(S[i], kt[i * LPC], d0);
          d1 = fmaf(S[i + 1], kt[(i + 1) * LPC], d1);
          d2 = fmaf(S[i + 2], kt[(i + 2) * LPC], d2);
          d3 = fmaf(S[i + 3], kt[(i + 3) * LPC], d3);
        }
        float dot = (d0 + d1) + (d2 + d3);
        for (int o = 1; o < LPC; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        u = bs[tt] * (vt - dot);
      } else {
        const float g = as[tt];
#pragma unroll
        for (int i = 0; i < RPL; ++i) S[i] *= g;
        u = bs[tt] * vt;
      }
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
      for (int i = 0; i < RPL; i += 4) {
        S[i] = fmaf(kt[i * LPC], u, S[i]);
        S[i + 1] = fmaf(kt[(i + 1) * LPC], u, S[i + 1]);
        S[i + 2] = fmaf(kt[(i + 2) * LPC], u, S[i + 2]);
        S[i + 3] = fmaf(kt[(i + 3) * LPC], u, S[i + 3]);
        o0 = fmaf(S[i], qt[i * LPC], o0);
        o1 = fmaf(S[i + 1], qt[(i + 1) * LPC], o1);
        o2 = fmaf(S[i + 2], qt[(i + 2) * LPC], o2);
        o3 = fmaf(S[i + 3], qt[(i + 3) * LPC], o3);
      }
      float o = (o0 + o1) + (o2 + o3);
      for (int off = 1; off < LPC; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (live && part == 0) a.out[(row0 + t0 + tt) * a.ldo + h * E + e] = fmaf(skip, vt, o);
    }
    __syncthreads();                           // this half may be staged again
  }
#pragma unroll
  for (int i = 0; i < RPL; ++i) {
    const int r = i * LPC + part;
    if (live && r < D) srow[static_cast<int64_t>(r) * E + e] = S[i];
  }
}

}  // namespace b200

extern "C" int b200_causal_conv_silu(const void* x, int64_t ldx, const float* w, const float* bias,
                                     float* state, int64_t ld_state, const int64_t* slot,
                                     const int* tok_pos, const int* tok_b, const int* ext_start,
                                     const int* ext_len, void* out, int64_t ldo, int T, int bs, int C,
                                     int taps, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(x && w && state && slot && tok_pos && tok_b && ext_start && ext_len && out,
               "b200_causal_conv_silu: null pointer");
  B200_REQUIRE(T > 0 && bs > 0 && C > 0 && taps >= 1 && ld_state >= static_cast<int64_t>(taps - 1) * C,
               "b200_causal_conv_silu: %d channels, %d taps, state row of %lld", C, taps,
               static_cast<long long>(ld_state));
  B200_REQUIRE(x != out, "b200_causal_conv_silu: the state update reads the inputs after the convolution");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("causal_conv_silu", st);
  const int cb = ceil_div(C, kConvThreads);
#define LAUNCH(TT)                                                                                   \
  do {                                                                                               \
    launch_kernel(causal_conv_silu_kernel<TT>, dim3(T, cb), dim3(kConvThreads), 0, st, 1, 0,        \
                  static_cast<const TT*>(x), ldx, w, bias, state, ld_state, slot, tok_pos, tok_b,    \
                  ext_start, static_cast<TT*>(out), ldo, C, taps);                                   \
    B200_CHECK_LAUNCH("causal_conv_silu_kernel");                                                   \
    if (taps > 1) {                                                                                  \
      launch_kernel(conv_state_update_kernel<TT>, dim3(bs, cb), dim3(kConvThreads), 0, st, 1, 0,    \
                    static_cast<const TT*>(x), ldx, state, ld_state, slot, tok_pos, ext_start,       \
                    ext_len, C, taps);                                                               \
      B200_CHECK_LAUNCH("conv_state_update_kernel");                                                \
    }                                                                                                \
  } while (0)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_causal_conv_silu: dtype %d", dtype);
#undef LAUNCH
  return 0;
}

extern "C" int64_t b200_delta_recurrence_state_width(int H, int D, int E) {
  return static_cast<int64_t>(H) * D * E;
}

extern "C" int64_t b200_delta_recurrence_work_width(int H, int G, int D, int mode) {
  return 2 * static_cast<int64_t>(G) * D + (mode == 0 ? static_cast<int64_t>(H) * D : 0) + 2 * H;
}

extern "C" int b200_delta_recurrence(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                     const void* v, int64_t ldv, const void* decay_raw,
                                     int64_t ld_decay, const float* decay_bias, const float* a_log,
                                     const void* beta_raw, int64_t ld_beta, const float* skip,
                                     float q_scale, float unit_eps, int mode, float* state,
                                     int64_t ld_state, const int64_t* slot, const int* tok_pos,
                                     const int* ext_start, const int* ext_len, float* out, int64_t ldo,
                                     float* work, int T, int bs, int H, int G, int D, int E, int dtype,
                                     void* stream) {
  using namespace b200;
  if (bs == 0 || T == 0) return 0;
  B200_REQUIRE(q && k && v && decay_raw && decay_bias && a_log && state && slot && tok_pos && ext_start &&
                   ext_len && out && work,
               "b200_delta_recurrence: null pointer");
  B200_REQUIRE(mode == 0 || mode == 1, "b200_delta_recurrence: mode %d", mode);
  B200_REQUIRE(mode == 1 || beta_raw, "b200_delta_recurrence: the delta rule needs its write strengths");
  B200_REQUIRE(bs > 0 && T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && D <= 1024 && E > 0 && H <= 65535,
               "b200_delta_recurrence: heads %d / %d, key rows %d, value columns %d", H, G, D, E);
  B200_REQUIRE(ld_state >= static_cast<int64_t>(H) * D * E, "b200_delta_recurrence: state row too short");
  B200_REQUIRE(aligned16(work), "b200_delta_recurrence: the workspace must be 16-byte aligned");
  const int rpl = D <= 16 ? 16 : 32;
  int lpc = 1;
  while (rpl * lpc < D) lpc <<= 1;
  // one or two warps per CTA: enough CTAs to fill the machine when few sequences are in the step
  int nt = 64;
  if (static_cast<int64_t>(bs) * H * ceil_div(E * lpc, 64) < 2 * device_sm_count()) nt = 32;
  const int cols = nt / lpc;
  const dim3 grid(bs, H, ceil_div(E, cols));
  const int Dp = rpl * lpc;
  int chunk = kDeltaChunk;
  auto smem_for = [&](int ch) {
    return sizeof(float) * 2 * ((static_cast<size_t>(ch) * Dp * (mode == 0 ? 3 : 2) + 2 * ch +
                                 static_cast<size_t>(ch) * cols + 3) & ~static_cast<size_t>(3));
  };
  while (chunk > 1 && smem_for(chunk) > 160 * 1024) chunk >>= 1;
  const size_t smem = smem_for(chunk);
  B200_REQUIRE(smem <= 200 * 1024, "b200_delta_recurrence: key rows %d too many", D);
  // workspace: kq [T, 2 G D] | g [T, H D] (delta rule) | ab [T, 2 H]; every part starts 16-byte aligned
  // when D is a multiple of 4 (the vector path of the scan)
  float* kq = work;
  float* g = kq + static_cast<int64_t>(T) * 2 * G * D;
  float* ab = g + (mode == 0 ? static_cast<int64_t>(T) * H * D : 0);
  DeltaArgs a{v, ldv, kq, g, ab, skip, state, ld_state, slot, tok_pos, ext_start, ext_len, out, ldo,
              H, G, D, E, lpc, chunk};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer(mode == 0 ? "delta_recurrence" : "ssm_recurrence", st);
#define PREP(TT, DL)                                                                                 \
  launch_kernel(delta_prepare_kernel<TT, DL>, dim3(T), dim3(256), 0, st, 1, 0,                      \
                static_cast<const TT*>(q), ldq, static_cast<const TT*>(k), ldk,                      \
                static_cast<const TT*>(decay_raw), ld_decay, decay_bias, a_log,                      \
                static_cast<const TT*>(beta_raw), ld_beta, q_scale, unit_eps, kq, g, ab, H, G, D)
#define LAUNCH3(TT, R, DL)                                                                           \
  do {                                                                                               \
    PREP(TT, DL);                                                                                    \
    B200_CHECK_LAUNCH("delta_prepare_kernel");                                                      \
    if (smem > 48 * 1024)                                                                            \
      B200_CUDA_OK(cudaFuncSetAttribute(delta_recurrence_kernel<TT, R, DL>,                          \
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));    \
    launch_kernel(delta_recurrence_kernel<TT, R, DL>, grid, dim3(nt), smem, st, 1, 0, a);            \
  } while (0)
#define LAUNCH(TT)                                                                                   \
  do {                                                                                               \
    if (rpl == 16 && mode == 0) LAUNCH3(TT, 16, true);                                               \
    else if (rpl == 16) LAUNCH3(TT, 16, false);                                                      \
    else if (mode == 0) LAUNCH3(TT, 32, true);                                                       \
    else LAUNCH3(TT, 32, false);                                                                     \
  } while (0)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_delta_recurrence: dtype %d", dtype);
#undef LAUNCH
#undef LAUNCH3
#undef PREP
  B200_CHECK_LAUNCH("delta_recurrence_kernel");
  return 0;
}
