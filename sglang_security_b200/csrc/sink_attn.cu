// Grouped-query softmax attention over a paged token pool whose row holds [keys | values] of all
// key/value heads, with the options of the designs that use it:
//   * RMS norm of the query and key projections over a group of coordinates (the whole projection, or
//     one head) with a learned weight, before rotation;
//   * rotary positions in the interleaved pairing on the first `rot_dims` coordinates of each head;
//   * a causal sliding window that also keeps the first `keep_first` tokens of the sequence visible
//     (at their true positions);
//   * a learned sink per query head: exp(sink) joins the softmax denominator, with no key or value;
//   * key size D and value size E that differ;
//   * a query temperature that grows with the position in steps: q *= 1 + coef * ln(floor((p + 1) / every) + 1);
//   * RMS norm of each value head (no weight), and a mix of the normed values with the values another
//     layer cached for the same token: v <- (1 - lambda) v + lambda v_first;
//   * a soft cap on the scaled scores: s <- cap * tanh(s / cap);
//   * the weights of every query head applied to the values of EVERY key/value head (one grid plane
//     per value head), for designs that mix the heads' weights after the softmax: the mixed output is
//     a linear combination of these per-head products (csrc/head_mix.cu).
//
//   qk_norm_rope_write : per token, from the projection outputs: q -> norm -> rotation -> fp32 queries;
//                        k -> norm -> rotation -> pool row; v -> pool row.  Norms and angles in fp32;
//                        the angle is position x frequency with the frequency held as a sum of two
//                        floats, so it is as exact at position 100000 as at position 10.
//   sink_attn          : one CTA per (token, key/value head); the query heads that share the key/value
//                        head are scored together, four per pass, so their keys and values are read
//                        once.  The CTA's 4 to 16 warps (by the longest key list) take the visible keys
//                        in tiles of 32: a lane scores one key against the pass's heads, then the warp
//                        accumulates the tile's values (4 columns per lane, several keys in flight), each
//                        warp with a running maximum and sum per head, merged in warp order at the end.
//                        Scores, weights and sums are fp32.  Every token walks its own list of visible
//                        keys through req_to_token, so prompt portions and decoded tokens of different
//                        requests mix freely in one launch; a token list restricts a launch to some rows.
#include <type_traits>

#include "common.cuh"

namespace b200 {

constexpr int kPrepThreads = 256;

__device__ __forceinline__ float prep_block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  float t = (l < kPrepThreads / 32) ? red[l] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// One projection row [heads * D] -> normed (groups of `group`, 0 = no norm) and rotated values.
// `inv` holds 1 / rms per group in shared memory.
template <typename T>
__device__ __forceinline__ float normed(const T* row, int idx, const float* w, const float* inv,
                                        int group) {
  float x = to_float<T>(row[idx]);
  if (group > 0) x *= inv[idx / group] * (w ? w[idx] : 1.f);
  return x;
}

template <typename T>
__device__ void group_inv_rms(const T* row, int n, int group, float eps, float* inv, float* red) {
  // few groups (the whole projection, or one per head): one block-wide sum per group
  for (int g = 0; g * group < n; ++g) {
    float s = 0.f;
    for (int d = threadIdx.x; d < group; d += kPrepThreads) {
      const float x = to_float<T>(row[g * group + d]);
      s = fmaf(x, x, s);
    }
    s = prep_block_sum(s, red);
    if (threadIdx.x == 0) inv[g] = 1.0f / sqrtf(s / static_cast<float>(group) + eps);
  }
  __syncthreads();
}

template <typename T, typename TP>
__global__ void __launch_bounds__(kPrepThreads)
qk_norm_rope_write_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                          const T* __restrict__ v, int64_t ldv, const float* __restrict__ qw,
                          const float* __restrict__ kw, int q_group, int k_group, float eps,
                          const float* __restrict__ freq_hi, const float* __restrict__ freq_lo,
                          int rot_dims, const int* __restrict__ tok_pos,
                          const int64_t* __restrict__ loc, TP* __restrict__ pool, int64_t ld_pool,
                          int k_off, int v_off, float* __restrict__ q_out, int64_t ldqo,
                          T* __restrict__ q_out16, int64_t ldqo16, int H, int G, int D, int E,
                          float temp_coef, int temp_every, int v_norm, const float* __restrict__ v_mix,
                          const TP* __restrict__ first_pool, int64_t ld_first, int first_off) {
  extern __shared__ float prep_smem[];       // [rot_dims / 2] cos, [rot_dims / 2] sin, group scales
  __shared__ float red[kPrepThreads / 32];
  const int t = blockIdx.x, half = rot_dims / 2;
  float* cs = prep_smem;
  float* sn = cs + half;
  float* inv_q = sn + half;
  float* inv_k = inv_q + (q_group > 0 ? (H * D) / q_group : 0);
  const float pos = static_cast<float>(tok_pos[t]);
  for (int i = threadIdx.x; i < half; i += kPrepThreads) {
    const float hi = freq_hi[i], lo = freq_lo ? freq_lo[i] : 0.f;
    const float a = pos * hi;
    const float err = fmaf(pos, hi, -a) + pos * lo;     // what the rounded product dropped
    float s, c;
    sincosf(a, &s, &c);
    cs[i] = c - err * s;
    sn[i] = s + err * c;
  }
  const T* qr = q + t * ldq;
  const T* kr = k + t * ldk;
  // query temperature: a step function of the position, fp32
  const float temp = temp_every > 0
                         ? 1.0f + temp_coef * logf(static_cast<float>((tok_pos[t] + 1) / temp_every) + 1.0f)
                         : 1.0f;
  if (q_group > 0) group_inv_rms(qr, H * D, q_group, eps, inv_q, red);
  if (k_group > 0) group_inv_rms(kr, G * D, k_group, eps, inv_k, red);
  __syncthreads();
  TP* prow = pool + loc[t] * ld_pool;
  for (int idx = threadIdx.x; idx < (H + G) * D; idx += kPrepThreads) {
    const bool is_q = idx < H * D;
    const int i = is_q ? idx : idx - H * D;
    const int d = i % D;
    const T* row = is_q ? qr : kr;
    const float* w = is_q ? qw : kw;
    const float* inv = is_q ? inv_q : inv_k;
    const int group = is_q ? q_group : k_group;
    float x = normed(row, i, w, inv, group);
    if (d < rot_dims) {
      const float y = normed(row, i - d + (d ^ 1), w, inv, group);   // rot_dims is even: the pair stays in the head
      const float c = cs[d >> 1], s = sn[d >> 1];
      x = (d & 1) ? fmaf(x, c, y * s) : fmaf(x, c, -y * s);
    }
    if (is_q) {
      x *= temp;
      if (q_out) q_out[t * ldqo + i] = x;
      if (q_out16) q_out16[t * ldqo16 + i] = from_float<T>(x);
    } else {
      prow[k_off + i] = from_float<TP>(x);
    }
  }
  const T* vr = v + t * ldv;
  if (!v_norm && !first_pool) {
    for (int i = threadIdx.x; i < G * E; i += kPrepThreads)
      prow[v_off + i] = from_float<TP>(to_float<T>(vr[i]));
    return;
  }
  // one warp per value head: unit RMS over the head (fp32), then the mix with the first layer's row
  const TP* first = first_pool ? first_pool + loc[t] * ld_first + first_off : nullptr;
  const float lam = (first && v_mix) ? *v_mix : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int g = warp; g < G; g += kPrepThreads / 32) {
    float inv = 1.f;
    if (v_norm) {
      float ss = 0.f;
      for (int e = lane; e < E; e += 32) {
        const float x = to_float<T>(vr[g * E + e]);
        ss = fmaf(x, x, ss);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      inv = 1.0f / sqrtf(ss / static_cast<float>(E) + eps);
    }
    for (int e = lane; e < E; e += 32) {
      float x = to_float<T>(vr[g * E + e]) * inv;
      if (first) x = (1.0f - lam) * x + lam * to_float<TP>(first[g * E + e]);
      prow[v_off + g * E + e] = from_float<TP>(x);
    }
  }
}

constexpr int kSinkMaxWarps = 16;  // warps per CTA: 4 to 16, by the longest key list (host)
constexpr int kSinkMaxCols = 8;    // value size <= 256
constexpr int kSinkHeads = 4;      // query heads of a key/value head scored per pass over its keys

template <typename TP, typename TO>
__global__ void __launch_bounds__(kSinkMaxWarps * 32)
sink_attn_kernel(const float* __restrict__ q, int64_t ldq, const TP* __restrict__ pool,
                 int64_t ld_pool, int k_off, int v_off, const int* __restrict__ req_to_token,
                 int64_t ld_r2t, const int64_t* __restrict__ req_idx, const int* __restrict__ tok_pos,
                 const int* __restrict__ tok_b, const float* __restrict__ sink, float scale, int window,
                 int keep_first, TO* __restrict__ out, int64_t ldo, int H, int G, int D, int E,
                 const int* __restrict__ tok_list, float softcap, int64_t ldo_plane) {
  extern __shared__ __align__(16) float sink_smem[];
  constexpr int RH = kSinkHeads;
  const int nw = blockDim.x >> 5;
  float* qs = sink_smem;                       // [RH][D] scaled queries of the pass
  float* wacc = qs + RH * D;                   // [nw][RH][E]
  float* wm = wacc + nw * RH * E;              // [nw][RH]
  float* wl = wm + nw * RH;                    // [nw][RH]
  float* wf = wl + nw * RH;                    // [nw][RH] merge factors
  float* wt = wf + nw * RH;                    // [RH] merged denominators
  const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, g = blockIdx.y, R = H / G;
  // value head: the key/value head's own, or (one grid plane per value head) plane z
  const int gv = gridDim.z > 1 ? static_cast<int>(blockIdx.z) : g;
  out += static_cast<int64_t>(blockIdx.z) * ldo_plane;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = tok_pos[t];
  const int* r2t = req_to_token + req_idx[tok_b[t]] * ld_r2t;
  // visible keys: the first `kf` positions, then lo .. p
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int kf = min(keep_first, lo);
  const int nkeys = kf + (p - lo + 1);
  const bool vec = (D % 8 == 0) && sizeof(TP) == 2 && (ld_pool % 8 == 0) && ((k_off + g * D) % 8 == 0) &&
                   ((reinterpret_cast<uintptr_t>(pool) & 15) == 0);
  // values: 4 consecutive columns per lane with vector loads when every piece is aligned
  const bool vblk = (E % 4 == 0) && (ld_pool % 4 == 0) && ((v_off + gv * E) % 4 == 0) &&
                    ((reinterpret_cast<uintptr_t>(pool) & 15) == 0);
  // the query heads that share this key/value head, RH at a time: their keys and values are read once
  // per pass
  for (int h0 = 0; h0 < R; h0 += RH) {
    const int nr = min(RH, R - h0), hb = g * R + h0;
    __syncthreads();                           // the previous pass has finished with the shared arrays
    for (int i = threadIdx.x; i < RH * D; i += blockDim.x) {
      const int r = i / D, d = i - r * D;
      qs[i] = r < nr ? q[t * ldq + (hb + r) * D + d] * scale : 0.f;
    }
    __syncthreads();
    float m[RH], l[RH], acc[RH][kSinkMaxCols];
#pragma unroll
    for (int r = 0; r < RH; ++r) {
      m[r] = -INFINITY;
      l[r] = 0.f;
#pragma unroll
      for (int c = 0; c < kSinkMaxCols; ++c) acc[r][c] = 0.f;
    }
    for (int n0 = warp * 32; n0 < nkeys; n0 += nw * 32) {
      const int n = n0 + lane;
      int64_t slot = 0;
      float s[RH];
#pragma unroll
      for (int r = 0; r < RH; ++r) s[r] = 0.f;
      if (n < nkeys) {
        const int j = n < kf ? n : lo + (n - kf);
        slot = r2t[j];
        const TP* kr = pool + slot * ld_pool + k_off + g * D;
        bool done = false;
        if constexpr (sizeof(TP) == 2) {
#pragma unroll 2
          for (int d = 0; vec && d < D; d += 8) {
            const uint4 u = *reinterpret_cast<const uint4*>(kr + d);
            const TP* e8 = reinterpret_cast<const TP*>(&u);
            float kv[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) kv[i] = to_float<TP>(e8[i]);
#pragma unroll
            for (int r = 0; r < RH; ++r) {
              const float4 q0 = *reinterpret_cast<const float4*>(qs + r * D + d);
              const float4 q1 = *reinterpret_cast<const float4*>(qs + r * D + d + 4);
              s[r] = fmaf(q0.x, kv[0], s[r]);
              s[r] = fmaf(q0.y, kv[1], s[r]);
              s[r] = fmaf(q0.z, kv[2], s[r]);
              s[r] = fmaf(q0.w, kv[3], s[r]);
              s[r] = fmaf(q1.x, kv[4], s[r]);
              s[r] = fmaf(q1.y, kv[5], s[r]);
              s[r] = fmaf(q1.z, kv[6], s[r]);
              s[r] = fmaf(q1.w, kv[7], s[r]);
            }
          }
          done = vec;
        }
        if (!done) {
          for (int d = 0; d < D; ++d) {
            const float kd = to_float<TP>(kr[d]);
#pragma unroll
            for (int r = 0; r < RH; ++r) s[r] = fmaf(qs[r * D + d], kd, s[r]);
          }
        }
      }
      if (softcap > 0.f) {
#pragma unroll
        for (int r = 0; r < RH; ++r) s[r] = softcap * tanhf(s[r] * inv_cap);
      }
      float pj[RH];
#pragma unroll
      for (int r = 0; r < RH; ++r) {
        const float sr = n < nkeys ? s[r] : -INFINITY;
        float tm = sr;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
        const float mn = fmaxf(m[r], tm);
        const float corr = expf(m[r] - mn);       // m = -inf on the first tile: exp(-inf) = 0
        pj[r] = n < nkeys ? expf(sr - mn) : 0.f;
        float ps = pj[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l[r] = l[r] * corr + ps;
        m[r] = mn;
#pragma unroll
        for (int c = 0; c < kSinkMaxCols; ++c) acc[r][c] *= corr;
      }
      const int cnt = min(32, nkeys - n0);
      if (vblk) {
        // a lane owns 4 consecutive columns per 128: one 8-byte (16-bit pool) or 16-byte load per key;
        // the rows of 8 keys are requested before the first is used (a loop that loads and uses one key
        // at a time waits a full memory round trip per key)
        using V4 = typename std::conditional<sizeof(TP) == 2, uint2, float4>::type;
#pragma unroll
        for (int c = 0; c < kSinkMaxCols / 4; ++c) {
          if (128 * c >= E) continue;            // the same for all lanes: they shuffle together below
          const int e = 128 * c + 4 * lane;
          const bool col_ok = e < E;
          for (int j0 = 0; j0 < cnt; j0 += 8) {
            V4 u[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int64_t sl = __shfl_sync(0xffffffffu, slot, (j0 + i) & 31);   // lanes past cnt hold slot 0
              u[i] = *reinterpret_cast<const V4*>(pool + sl * ld_pool + v_off + gv * E + (col_ok ? e : 0));
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              float x[4];
              if constexpr (sizeof(TP) == 2) {
                const TP* t4 = reinterpret_cast<const TP*>(&u[i]);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) x[k4] = to_float<TP>(t4[k4]);
              } else {
                const float* f4 = reinterpret_cast<const float*>(&u[i]);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) x[k4] = f4[k4];
              }
              const bool live = col_ok && j0 + i < cnt;
#pragma unroll
              for (int r = 0; r < RH; ++r) {
                const float pw = __shfl_sync(0xffffffffu, pj[r], (j0 + i) & 31);
                if (live) {
#pragma unroll
                  for (int k4 = 0; k4 < 4; ++k4) acc[r][4 * c + k4] = fmaf(pw, x[k4], acc[r][4 * c + k4]);
                }
              }
            }
          }
        }
      } else {
        for (int jj = 0; jj < cnt; ++jj) {
          const int64_t sl = __shfl_sync(0xffffffffu, slot, jj);
          float pw[RH];
#pragma unroll
          for (int r = 0; r < RH; ++r) pw[r] = __shfl_sync(0xffffffffu, pj[r], jj);
          const TP* vr = pool + sl * ld_pool + v_off + gv * E;
#pragma unroll
          for (int c = 0; c < kSinkMaxCols; ++c) {
            const int e = lane + 32 * c;
            if (e < E) {
              const float x = to_float<TP>(vr[e]);
#pragma unroll
              for (int r = 0; r < RH; ++r) acc[r][c] = fmaf(pw[r], x, acc[r][c]);
            }
          }
        }
      }
    }
    // per-warp partial softmaxes -> shared memory, merged in warp order
#pragma unroll
    for (int r = 0; r < RH; ++r) {
      if (lane == 0) {
        wm[warp * RH + r] = m[r];
        wl[warp * RH + r] = l[r];
      }
#pragma unroll
      for (int c = 0; c < kSinkMaxCols; ++c) {
        const int e = vblk ? 128 * (c / 4) + 4 * lane + (c & 3) : lane + 32 * c;
        if (e < E) wacc[(warp * RH + r) * E + e] = acc[r][c];
      }
    }
    __syncthreads();
    if (threadIdx.x < nr) {
      const int r = threadIdx.x;
      float mt = sink ? sink[hb + r] : -INFINITY;
      for (int w = 0; w < nw; ++w) mt = fmaxf(mt, wm[w * RH + r]);
      float lt = sink ? expf(sink[hb + r] - mt) : 0.f;
      for (int w = 0; w < nw; ++w) {
        const float f = wm[w * RH + r] == -INFINITY ? 0.f : expf(wm[w * RH + r] - mt);
        wf[w * RH + r] = f;
        lt = fmaf(wl[w * RH + r], f, lt);
      }
      wt[r] = lt;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nr * E; i += blockDim.x) {
      const int r = i / E, e = i - r * E;
      float o = 0.f;
      for (int w = 0; w < nw; ++w) o = fmaf(wacc[(w * RH + r) * E + e], wf[w * RH + r], o);
      out[t * ldo + (hb + r) * E + e] = from_float<TO>(o / wt[r]);
    }
  }
}

}  // namespace b200

extern "C" int b200_qkv_prep_write(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                   const void* v, int64_t ldv, const float* qw, const float* kw,
                                   int q_group, int k_group, float eps, const float* freq_hi,
                                   const float* freq_lo, int rot_dims, const int* tok_pos,
                                   const int64_t* loc, void* pool, int64_t ld_pool, int k_off,
                                   int v_off, float* q_out, int64_t ldqo, void* q_out16,
                                   int64_t ldqo16, int T, int H, int G, int D, int E, float temp_coef,
                                   int temp_every, int v_norm, const float* v_mix,
                                   const void* first_pool, int64_t ld_first, int first_off, int dtype,
                                   void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(q && k && v && tok_pos && loc && pool && (q_out || q_out16),
               "b200_qkv_prep_write: null pointer");
  B200_REQUIRE(T > 0 && H > 0 && G > 0 && D > 0 && E > 0 && rot_dims >= 0 && rot_dims <= D &&
                   rot_dims % 2 == 0 && (rot_dims == 0 || freq_hi),
               "b200_qkv_prep_write: head size %d, rotated %d", D, rot_dims);
  B200_REQUIRE((q_group == 0 || (H * D) % q_group == 0) && (k_group == 0 || (G * D) % k_group == 0) &&
                   q_group >= 0 && k_group >= 0,
               "b200_qkv_prep_write: norm groups %d / %d do not divide the projections", q_group,
               k_group);
  B200_REQUIRE(temp_every >= 0 && (!first_pool || v_mix),
               "b200_qkv_prep_write: temperature step %d; a value mix needs its weight", temp_every);
  const size_t smem = sizeof(float) * (rot_dims + (q_group ? H * D / q_group : 0) +
                                       (k_group ? G * D / k_group : 0) + 1);
  B200_REQUIRE(smem <= 48 * 1024, "b200_qkv_prep_write: too many norm groups");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("qk_norm_rope_write", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(qk_norm_rope_write_kernel<TT, TT>, dim3(T), dim3(kPrepThreads), smem, st, 1, 0,      \
                static_cast<const TT*>(q), ldq, static_cast<const TT*>(k), ldk,                      \
                static_cast<const TT*>(v), ldv, qw, kw, q_group, k_group, eps, freq_hi, freq_lo,     \
                rot_dims, tok_pos, loc, static_cast<TT*>(pool), ld_pool, k_off, v_off, q_out, ldqo,  \
                static_cast<TT*>(q_out16), ldqo16, H, G, D, E, temp_coef, temp_every, v_norm, v_mix, \
                static_cast<const TT*>(first_pool), ld_first, first_off)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_qkv_prep_write: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("qk_norm_rope_write_kernel");
  return 0;
}

extern "C" int b200_qk_norm_rope_write(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                       const void* v, int64_t ldv, const float* qw, const float* kw,
                                       int q_group, int k_group, float eps, const float* freq_hi,
                                       const float* freq_lo, int rot_dims, const int* tok_pos,
                                       const int64_t* loc, void* pool, int64_t ld_pool, int k_off,
                                       int v_off, float* q_out, int64_t ldqo, void* q_out16,
                                       int64_t ldqo16, int T, int H, int G, int D, int E, int dtype,
                                       void* stream) {
  return b200_qkv_prep_write(q, ldq, k, ldk, v, ldv, qw, kw, q_group, k_group, eps, freq_hi, freq_lo,
                             rot_dims, tok_pos, loc, pool, ld_pool, k_off, v_off, q_out, ldqo, q_out16,
                             ldqo16, T, H, G, D, E, 0.f, 0, 0, nullptr, nullptr, 0, 0, dtype, stream);
}

// softcap > 0: scores are capped (cap * tanh(s / cap)) before the softmax.  all_values != 0: the weights
// of every query head are applied to the values of every key/value head; `out` is then fp32
// [G planes][T rows of ldo][H, E] with `ldo_plane` elements between planes.
extern "C" int b200_sink_attn_heads(const float* q, int64_t ldq, const void* pool, int64_t ld_pool,
                                    int k_off, int v_off, const int* req_to_token, int64_t ld_r2t,
                                    const int64_t* req_idx, const int* tok_pos, const int* tok_b,
                                    const float* sink, float scale, float softcap, int window,
                                    int keep_first, void* out, int64_t ldo, int all_values,
                                    int64_t ldo_plane, int T, int H, int G, int D, int E,
                                    const int* tok_list, int max_keys, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(q && pool && req_to_token && req_idx && tok_pos && tok_b && out,
               "b200_sink_attn: null pointer");
  B200_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && E > 0 && E <= 32 * kSinkMaxCols &&
                   window >= 0 && keep_first >= 0 && G <= 65535 && softcap >= 0.f,
               "b200_sink_attn: heads %d / %d, key size %d, value size %d (max %d)", H, G, D, E,
               32 * kSinkMaxCols);
  // one warp per 64 keys of the longest list (a hint; 0 = unknown): a warp's tiles are dependent round
  // trips to memory (slots, keys, values), so long lists want many warps and short ones few
  int nw = max_keys <= 0 ? 4 : min(kSinkMaxWarps, max(4, ceil_div(max_keys, 64)));
  auto smem_for = [&](int w) {
    return sizeof(float) * (static_cast<size_t>(kSinkHeads) * D + static_cast<size_t>(w) * kSinkHeads * (E + 3) +
                            kSinkHeads + 4);
  };
  while (nw > 1 && smem_for(nw) > 48 * 1024) nw >>= 1;
  const size_t smem = smem_for(nw);
  B200_REQUIRE(smem <= 48 * 1024, "b200_sink_attn: key size %d too large", D);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("sink_attn", st);
  const dim3 grid(T, G, all_values && G > 1 ? G : 1);
  if (!(all_values && G > 1)) ldo_plane = 0;
#define LAUNCH(TT, TO)                                                                               \
  launch_kernel(sink_attn_kernel<TT, TO>, grid, dim3(nw * 32), smem, st, 1, 0, q, ldq,               \
                static_cast<const TT*>(pool), ld_pool, k_off, v_off, req_to_token, ld_r2t, req_idx,  \
                tok_pos, tok_b, sink, scale, window, keep_first, static_cast<TO*>(out), ldo, H, G, D, \
                E, tok_list, softcap, ldo_plane)
  if (all_values) {
    if (dtype == B200_BF16) LAUNCH(__nv_bfloat16, float);
    else if (dtype == B200_F16) LAUNCH(__half, float);
    else if (dtype == B200_F32) LAUNCH(float, float);
    else B200_REQUIRE(false, "b200_sink_attn: dtype %d", dtype);
  } else {
    if (dtype == B200_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
    else if (dtype == B200_F16) LAUNCH(__half, __half);
    else if (dtype == B200_F32) LAUNCH(float, float);
    else B200_REQUIRE(false, "b200_sink_attn: dtype %d", dtype);
  }
#undef LAUNCH
  B200_CHECK_LAUNCH("sink_attn_kernel");
  return 0;
}

extern "C" int b200_sink_attn(const float* q, int64_t ldq, const void* pool, int64_t ld_pool, int k_off,
                              int v_off, const int* req_to_token, int64_t ld_r2t,
                              const int64_t* req_idx, const int* tok_pos, const int* tok_b,
                              const float* sink, float scale, int window, int keep_first, void* out,
                              int64_t ldo, int T, int H, int G, int D, int E, const int* tok_list,
                              int max_keys, int dtype, void* stream) {
  return b200_sink_attn_heads(q, ldq, pool, ld_pool, k_off, v_off, req_to_token, ld_r2t, req_idx,
                              tok_pos, tok_b, sink, scale, 0.f, window, keep_first, out, ldo, 0, 0, T, H,
                              G, D, E, tok_list, max_keys, dtype, stream);
}
