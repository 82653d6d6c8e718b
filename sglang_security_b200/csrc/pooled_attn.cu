// Grouped-query softmax attention over a causal sliding window PLUS one pooled key and value per block
// of `P` tokens that lies wholly before the window, over the paged one-row-per-token pool
// ([keys | values] of all key/value heads), with rotated values:
//   * RMS norm of every query and key head over its own coordinates with one learned weight [D] shared
//     by the heads, before rotation;
//   * rotary positions on the first `rot_dims` coordinates of a head, in either pairing
//     (0: neighbours 2i, 2i+1; 1: halves i, i + rot_dims/2), angle = position * f_i;
//   * values rotated by their own position over all E coordinates (same pairing, own frequency table)
//     before they are cached; the attention's output at position p is turned back by -p, so that a
//     value enters the sum rotated by the distance only;
//   * a multiplier per query head on the scores (folded into the fp32 queries);
//   * a query at position p sees the tokens j with 0 <= p - j < window and the blocks b with
//     b * P + P - 1 <= p - window, i.e. the first lo / P blocks, lo = max(0, p - window + 1); a block's
//     key and value are the means of its P cached rows.  Tokens and blocks share one softmax.
//
//   headnorm_rot_write : per token, from the projection outputs: q -> norm -> rotation -> * head scale ->
//                        fp32 queries; k -> norm -> rotation -> pool row; v -> rotation -> pool row.
//   pool_block_means   : for every new token that completes a block, the fp32 mean of the block's P pool
//                        rows (read back from the pool through req_to_token, so it does not matter in how
//                        many steps the block arrived) -> row `slot of the block's last token / div` of
//                        the summary buffer (div = P when P divides the page size, else 1).
//   pooled_window_attn : one CTA per (token, key/value head); its query heads are scored together, four
//                        per pass; warps take the visible keys (blocks first, then tokens) in tiles of
//                        32: a lane scores one key, then the warp accumulates the tile's values, each
//                        warp with a running maximum and sum per head, merged in warp order.  Scores,
//                        weights, sums and the final counter-rotation are fp32.  In its `part` form it
//                        takes the blocks only and writes the normalised fp32 sum with the log2 of its
//                        denominator, for rows whose tokens were summed by the tensor-core kernel.
//   pooled_merge_unrotate : for the rows of long prompt portions: out = w1 * (window part, 16-bit, from the
//                        tcgen05 extend kernel with its row log-sums) + w2 * (block part, fp32), the weights
//                        from the two log-sums (one softmax over both key sets), then the counter-rotation.
#include <type_traits>

#include "common.cuh"

namespace b200 {

constexpr int kPoolPrepThreads = 256;

// cos / sin of position * frequency, the frequency given as a sum of two floats: the product's
// rounding error and the low part correct the result to first order
__device__ __forceinline__ void exact_sincos(float pos, float hi, float lo, float* c, float* s) {
  const float a = pos * hi;
  const float err = fmaf(pos, hi, -a) + pos * lo;
  float sn, cs;
  sincosf(a, &sn, &cs);
  *c = cs - err * sn;
  *s = sn + err * cs;
}

// partner coordinate, frequency index and sign of the sine term of coordinate d among `dims` rotated ones
__device__ __forceinline__ void rot_pair(int d, int dims, int pairing, int* partner, int* fi, float* sign) {
  if (pairing == 1) {
    const int half = dims >> 1;
    const bool first = d < half;
    *partner = first ? d + half : d - half;
    *fi = first ? d : d - half;
    *sign = first ? -1.f : 1.f;
  } else {
    *partner = d ^ 1;
    *fi = d >> 1;
    *sign = (d & 1) ? 1.f : -1.f;
  }
}

template <typename T>
__global__ void __launch_bounds__(kPoolPrepThreads)
headnorm_rot_write_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                          const T* __restrict__ v, int64_t ldv, const float* __restrict__ qw,
                          const float* __restrict__ kw, float eps, const float* __restrict__ freq_hi,
                          const float* __restrict__ freq_lo, int rot_dims,
                          const float* __restrict__ vfreq_hi, const float* __restrict__ vfreq_lo,
                          int pairing, const float* __restrict__ head_scale,
                          const int* __restrict__ tok_pos, const int64_t* __restrict__ loc,
                          T* __restrict__ pool, int64_t ld_pool, int k_off, int v_off,
                          float* __restrict__ q_out, int64_t ldqo, T* __restrict__ q_out16,
                          int64_t ldqo16, int H, int G, int D, int E) {
  extern __shared__ float pp_smem[];
  const int t = blockIdx.x, half = rot_dims / 2, vhalf = vfreq_hi ? E / 2 : 0;
  float* cs = pp_smem;              // [half]
  float* sn = cs + half;            // [half]
  float* vcs = sn + half;           // [vhalf]
  float* vsn = vcs + vhalf;         // [vhalf]
  float* inv = vsn + vhalf;         // [H + G] 1 / rms of every query head, then every key head
  const float pos = static_cast<float>(tok_pos[t]);
  for (int i = threadIdx.x; i < half; i += kPoolPrepThreads)
    exact_sincos(pos, freq_hi[i], freq_lo ? freq_lo[i] : 0.f, cs + i, sn + i);
  for (int i = threadIdx.x; i < vhalf; i += kPoolPrepThreads)
    exact_sincos(pos, vfreq_hi[i], vfreq_lo ? vfreq_lo[i] : 0.f, vcs + i, vsn + i);
  const T* qr = q + t * ldq;
  const T* kr = k + t * ldk;
  const T* vr = v + t * ldv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int hd = warp; hd < H + G; hd += kPoolPrepThreads / 32) {
    const T* row = hd < H ? qr + hd * D : kr + (hd - H) * D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) {
      const float x = to_float<T>(row[d]);
      ss = fmaf(x, x, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) inv[hd] = (hd < H ? qw : kw) ? 1.0f / sqrtf(ss / static_cast<float>(D) + eps) : 1.f;
  }
  __syncthreads();
  T* prow = pool + loc[t] * ld_pool;
  for (int idx = threadIdx.x; idx < (H + G) * D; idx += kPoolPrepThreads) {
    const bool is_q = idx < H * D;
    const int i = is_q ? idx : idx - H * D;
    const int hd = i / D, d = i - hd * D;
    const T* row = is_q ? qr : kr;
    const float* w = is_q ? qw : kw;
    const float r = inv[is_q ? hd : H + hd];
    float x = to_float<T>(row[i]) * r * (w ? w[d] : 1.f);
    if (d < rot_dims) {
      int pd, fi;
      float sg;
      rot_pair(d, rot_dims, pairing, &pd, &fi, &sg);
      const float y = to_float<T>(row[hd * D + pd]) * r * (w ? w[pd] : 1.f);
      x = fmaf(x, cs[fi], sg * y * sn[fi]);
    }
    if (is_q) {
      if (head_scale) x *= head_scale[hd];
      q_out[t * ldqo + i] = x;
      if (q_out16) q_out16[t * ldqo16 + i] = from_float<T>(x);
    } else {
      prow[k_off + i] = from_float<T>(x);
    }
  }
  for (int i = threadIdx.x; i < G * E; i += kPoolPrepThreads) {
    const int g = i / E, d = i - g * E;
    float x = to_float<T>(vr[i]);
    if (vhalf) {
      int pd, fi;
      float sg;
      rot_pair(d, E, pairing, &pd, &fi, &sg);
      x = fmaf(x, vcs[fi], sg * to_float<T>(vr[g * E + pd]) * vsn[fi]);
    }
    prow[v_off + i] = from_float<T>(x);
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
pool_block_means_kernel(const T* __restrict__ pool, int64_t ld_pool, int width,
                        float* __restrict__ pooled, int64_t ld_pooled, int P, int pdiv,
                        const int* __restrict__ req_to_token, int64_t ld_r2t,
                        const int64_t* __restrict__ req_idx, const int* __restrict__ tok_pos,
                        const int* __restrict__ tok_b) {
  const int t = blockIdx.x, p = tok_pos[t];
  if ((p + 1) % P) return;                       // this token does not complete a block
  const int* r2t = req_to_token + req_idx[tok_b[t]] * ld_r2t;
  float* dst = pooled + static_cast<int64_t>(r2t[p] / pdiv) * ld_pooled;
  const float invp = 1.0f / static_cast<float>(P);
  for (int col = threadIdx.x; col < width; col += 128) {
    float s = 0.f;
    for (int i = 0; i < P; ++i) s += to_float<T>(pool[static_cast<int64_t>(r2t[p - P + 1 + i]) * ld_pool + col]);
    dst[col] = s * invp;
  }
}

// acc[r][4 c + k] += weight_r(key) * row(key)[col_off + 128 c + 4 lane + k] over the `cnt` keys of a tile
// whose rows are row_index(lane) of `base`; weights and row indices are held one key per lane.
template <typename TR, int RH>
__device__ __forceinline__ void accumulate_rows(const TR* __restrict__ base, int64_t ld, int col_off, int E,
                                                int cnt, int64_t rowi, const float (&pj)[RH],
                                                float (&acc)[RH][8], int lane) {
  using V4 = typename std::conditional<sizeof(TR) == 2, uint2, float4>::type;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    if (128 * c >= E) continue;                // the same for all lanes: they shuffle together below
    const int e = 128 * c + 4 * lane;
    const bool col_ok = e < E;
    for (int j0 = 0; j0 < cnt; j0 += 8) {
      V4 u[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int64_t ri = __shfl_sync(0xffffffffu, rowi, (j0 + i) & 31);   // lanes past cnt hold row 0
        u[i] = *reinterpret_cast<const V4*>(base + ri * ld + col_off + (col_ok ? e : 0));
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        float x[4];
        if constexpr (sizeof(TR) == 2) {
          const TR* t4 = reinterpret_cast<const TR*>(&u[i]);
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) x[k4] = to_float<TR>(t4[k4]);
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
}

constexpr int kPwMaxWarps = 16;
constexpr int kPwMaxCols = 8;     // value size <= 256
constexpr int kPwHeads = 4;       // query heads of a key/value head scored per pass

template <typename TP, typename TO>
__global__ void __launch_bounds__(kPwMaxWarps * 32)
pooled_window_attn_kernel(const float* __restrict__ q, int64_t ldq, const TP* __restrict__ pool,
                          int64_t ld_pool, int k_off, int v_off, const float* __restrict__ pooled,
                          int64_t ld_pooled, int P, int pdiv, const int* __restrict__ req_to_token,
                          int64_t ld_r2t, const int64_t* __restrict__ req_idx,
                          const int* __restrict__ tok_pos, const int* __restrict__ tok_b, float scale,
                          int window, const float* __restrict__ vfreq_hi,
                          const float* __restrict__ vfreq_lo, int pairing, TO* __restrict__ out,
                          int64_t ldo, int H, int G, int D, int E, const int* __restrict__ tok_list,
                          float* __restrict__ part_out, int64_t ld_part, float* __restrict__ part_lse,
                          int64_t ld_lse) {
  extern __shared__ __align__(16) float pw_smem[];
  constexpr int RH = kPwHeads;
  const int nw = blockDim.x >> 5;
  float* qs = pw_smem;                         // [RH][D] scaled queries of the pass
  float* wacc = qs + RH * D;                   // [nw][RH][E]
  float* wm = wacc + nw * RH * E;              // [nw][RH]
  float* wl = wm + nw * RH;                    // [nw][RH]
  float* wf = wl + nw * RH;                    // [nw][RH] merge factors
  float* wt = wf + nw * RH;                    // [RH] merged denominators
  float* om = wt + RH;                         // [RH][E] merged outputs before the counter-rotation
  float* vcs = om + RH * E;                    // [E / 2]
  float* vsn = vcs + E / 2;                    // [E / 2]
  const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x, g = blockIdx.y, R = H / G;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int p = tok_pos[t];
  const int* r2t = req_to_token + req_idx[tok_b[t]] * ld_r2t;
  const int lo = window > 0 ? max(0, p - window + 1) : 0;
  const int npool = (pooled && P > 0) ? lo / P : 0;       // blocks that end before the window
  const int ntok = part_out ? 0 : p - lo + 1;                  // the part form takes the blocks only
  const int pool_tiles = (npool + 31) >> 5, tok_tiles = (ntok + 31) >> 5;
  if (part_out && npool == 0) {                // no block in sight: nothing to add to the window's part
    for (int i = threadIdx.x; i < R; i += blockDim.x) part_lse[t * ld_lse + g * R + i] = -INFINITY;
    return;
  }
  if (vfreq_hi && !part_out)
    for (int i = threadIdx.x; i < E / 2; i += blockDim.x)
      exact_sincos(static_cast<float>(p), vfreq_hi[i], vfreq_lo ? vfreq_lo[i] : 0.f, vcs + i, vsn + i);
  const bool kvec = sizeof(TP) == 2 && (D % 8 == 0) && (ld_pool % 8 == 0) && ((k_off + g * D) % 8 == 0) &&
                    ((reinterpret_cast<uintptr_t>(pool) & 15) == 0);
  const bool pvec = (D % 4 == 0) && (ld_pooled % 4 == 0) && ((k_off + g * D) % 4 == 0) &&
                    ((reinterpret_cast<uintptr_t>(pooled) & 15) == 0);
  // values in vector loads when every piece of both buffers is aligned (one column layout for both)
  const bool vblk = (E % 4 == 0) && (ld_pool % 4 == 0) && ((v_off + g * E) % 4 == 0) &&
                    ((reinterpret_cast<uintptr_t>(pool) & 15) == 0) &&
                    (!pooled || ((ld_pooled % 4 == 0) && (reinterpret_cast<uintptr_t>(pooled) & 15) == 0));
  for (int h0 = 0; h0 < R; h0 += RH) {
    const int nr = min(RH, R - h0), hb = g * R + h0;
    __syncthreads();
    for (int i = threadIdx.x; i < RH * D; i += blockDim.x) {
      const int r = i / D, d = i - r * D;
      qs[i] = r < nr ? q[t * ldq + (hb + r) * D + d] * scale : 0.f;
    }
    __syncthreads();
    float m[RH], l[RH], acc[RH][kPwMaxCols];
#pragma unroll
    for (int r = 0; r < RH; ++r) {
      m[r] = -INFINITY;
      l[r] = 0.f;
#pragma unroll
      for (int c = 0; c < kPwMaxCols; ++c) acc[r][c] = 0.f;
    }
    // blocks and tokens are walked in tiles of 32 that never mix the two (the blocks' last tile may be
    // partly filled), so a tile's rows have one type and one buffer
    for (int tile = warp; tile < pool_tiles + tok_tiles; tile += nw) {
      const bool is_pool = tile < pool_tiles;
      const int n = (is_pool ? tile : tile - pool_tiles) * 32 + lane;      // index within its kind
      const int cnt = min(32, (is_pool ? npool : ntok) - (n - lane));
      const bool have = lane < cnt;
      int64_t rowi = 0;                         // pool slot, or row of the summary buffer
      float s[RH];
#pragma unroll
      for (int r = 0; r < RH; ++r) s[r] = 0.f;
      if (have) {
        if (is_pool) {
          rowi = r2t[n * P + P - 1] / pdiv;
          const float* kp = pooled + rowi * ld_pooled + k_off + g * D;
          if (pvec) {
            for (int d = 0; d < D; d += 4) {
              const float4 kv = *reinterpret_cast<const float4*>(kp + d);
#pragma unroll
              for (int r = 0; r < RH; ++r) {
                const float4 q0 = *reinterpret_cast<const float4*>(qs + r * D + d);
                s[r] = fmaf(q0.x, kv.x, s[r]);
                s[r] = fmaf(q0.y, kv.y, s[r]);
                s[r] = fmaf(q0.z, kv.z, s[r]);
                s[r] = fmaf(q0.w, kv.w, s[r]);
              }
            }
          } else {
            for (int d = 0; d < D; ++d) {
              const float kd = kp[d];
#pragma unroll
              for (int r = 0; r < RH; ++r) s[r] = fmaf(qs[r * D + d], kd, s[r]);
            }
          }
        } else {
          rowi = r2t[lo + n];
          const TP* kr = pool + rowi * ld_pool + k_off + g * D;
          bool done = false;
          if constexpr (sizeof(TP) == 2) {
#pragma unroll 2
            for (int d = 0; kvec && d < D; d += 8) {
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
            done = kvec;
          }
          if (!done) {
            for (int d = 0; d < D; ++d) {
              const float kd = to_float<TP>(kr[d]);
#pragma unroll
              for (int r = 0; r < RH; ++r) s[r] = fmaf(qs[r * D + d], kd, s[r]);
            }
          }
        }
      }
      float pj[RH];
#pragma unroll
      for (int r = 0; r < RH; ++r) {
        const float sr = have ? s[r] : -INFINITY;
        float tm = sr;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, o));
        const float mn = fmaxf(m[r], tm);
        const float corr = expf(m[r] - mn);
        pj[r] = have ? expf(sr - mn) : 0.f;
        float ps = pj[r];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
        l[r] = l[r] * corr + ps;
        m[r] = mn;
#pragma unroll
        for (int c = 0; c < kPwMaxCols; ++c) acc[r][c] *= corr;
      }
      if (vblk) {
        // a lane owns 4 consecutive columns per 128: one 8-byte (16-bit rows) or 16-byte (fp32 rows) load
        // per key; the rows of 8 keys are requested before the first is used
        if (is_pool) accumulate_rows<float, RH>(pooled, ld_pooled, v_off + g * E, E, cnt, rowi, pj, acc, lane);
        else accumulate_rows<TP, RH>(pool, ld_pool, v_off + g * E, E, cnt, rowi, pj, acc, lane);
      } else {
        for (int jj = 0; jj < cnt; ++jj) {
          const int64_t ri = __shfl_sync(0xffffffffu, rowi, jj);
          float pw[RH];
#pragma unroll
          for (int r = 0; r < RH; ++r) pw[r] = __shfl_sync(0xffffffffu, pj[r], jj);
#pragma unroll
          for (int c = 0; c < kPwMaxCols; ++c) {
            const int e = lane + 32 * c;
            if (e < E) {
              const float x = is_pool ? pooled[ri * ld_pooled + v_off + g * E + e]
                                      : to_float<TP>(pool[ri * ld_pool + v_off + g * E + e]);
#pragma unroll
              for (int r = 0; r < RH; ++r) acc[r][c] = fmaf(pw[r], x, acc[r][c]);
            }
          }
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RH; ++r) {
      if (lane == 0) {
        wm[warp * RH + r] = m[r];
        wl[warp * RH + r] = l[r];
      }
#pragma unroll
      for (int c = 0; c < kPwMaxCols; ++c) {
        const int e = vblk ? 128 * (c / 4) + 4 * lane + (c & 3) : lane + 32 * c;
        if (e < E) wacc[(warp * RH + r) * E + e] = acc[r][c];
      }
    }
    __syncthreads();
    if (threadIdx.x < nr) {
      const int r = threadIdx.x;
      float mt = -INFINITY;
      for (int w = 0; w < nw; ++w) mt = fmaxf(mt, wm[w * RH + r]);
      float lt = 0.f;
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
      om[i] = wt[r] > 0.f ? o / wt[r] : 0.f;
    }
    __syncthreads();
    if (part_out) {
      // the normalised sum over the blocks and log2 of its denominator (-inf: no block in sight)
      for (int i = threadIdx.x; i < nr * E; i += blockDim.x)
        part_out[t * ld_part + hb * E + i] = om[i];
      if (threadIdx.x < nr) {
        const int r = threadIdx.x;
        float mt = -INFINITY;
        for (int w = 0; w < nw; ++w) mt = fmaxf(mt, wm[w * RH + r]);
        part_lse[t * ld_lse + hb + r] = wt[r] > 0.f ? (mt + logf(wt[r])) * 1.4426950408889634f : -INFINITY;
      }
      continue;
    }
    for (int i = threadIdx.x; i < nr * E; i += blockDim.x) {
      const int r = i / E, e = i - r * E;
      float o = om[i];
      if (vfreq_hi) {                           // turn back by the query's position: the angle's sign flips
        int pd, fi;
        float sg;
        rot_pair(e, E, pairing, &pd, &fi, &sg);
        o = fmaf(o, vcs[fi], -sg * om[r * E + pd] * vsn[fi]);
      }
      out[t * ldo + (hb + r) * E + e] = from_float<TO>(o);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
pooled_merge_unrotate_kernel(T* __restrict__ out, int64_t ldo, const float* __restrict__ lse1, int64_t ld1,
                             const float* __restrict__ part, int64_t ld_part,
                             const float* __restrict__ lse2, int64_t ld2,
                             const float* __restrict__ vfreq_hi, const float* __restrict__ vfreq_lo,
                             int pairing, const int* __restrict__ tok_pos,
                             const int* __restrict__ tok_list, int H, int E) {
  extern __shared__ float mg_smem[];          // [H * E] merged row, [E / 2] cos, [E / 2] sin
  float* row = mg_smem;
  float* vcs = row + H * E;
  float* vsn = vcs + E / 2;
  const int t = tok_list ? tok_list[blockIdx.x] : blockIdx.x;
  if (vfreq_hi)
    for (int i = threadIdx.x; i < E / 2; i += blockDim.x)
      exact_sincos(static_cast<float>(tok_pos[t]), vfreq_hi[i], vfreq_lo ? vfreq_lo[i] : 0.f, vcs + i, vsn + i);
  for (int i = threadIdx.x; i < H * E; i += blockDim.x) {
    const int h = i / E;
    float o = to_float<T>(out[t * ldo + i]);
    if (part) {
      // both parts are normalised sums; exp2 of their log-sums are the two denominators
      const float a = lse1[t * ld1 + h], b = lse2[t * ld2 + h];
      if (b != -INFINITY) {
        const float mx = fmaxf(a, b);
        const float wa = exp2f(a - mx), wb = exp2f(b - mx);
        o = (wa * o + wb * part[t * ld_part + i]) / (wa + wb);
      }
    }
    row[i] = o;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < H * E; i += blockDim.x) {
    const int h = i / E, e = i - h * E;
    float o = row[i];
    if (vfreq_hi) {
      int pd, fi;
      float sg;
      rot_pair(e, E, pairing, &pd, &fi, &sg);
      o = fmaf(o, vcs[fi], -sg * row[h * E + pd] * vsn[fi]);
    }
    out[t * ldo + i] = from_float<T>(o);
  }
}

}  // namespace b200

extern "C" int b200_headnorm_rot_write(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                       const void* v, int64_t ldv, const float* qw, const float* kw,
                                       float eps, const float* freq_hi, const float* freq_lo,
                                       int rot_dims, const float* vfreq_hi, const float* vfreq_lo,
                                       int pairing, const float* head_scale, const int* tok_pos,
                                       const int64_t* loc, void* pool, int64_t ld_pool, int k_off,
                                       int v_off, float* q_out, int64_t ldqo, void* q_out16,
                                       int64_t ldqo16, int T, int H, int G, int D, int E, int dtype,
                                       void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(q && k && v && tok_pos && loc && pool && q_out, "b200_headnorm_rot_write: null pointer");
  B200_REQUIRE(T > 0 && H > 0 && G > 0 && D > 0 && E > 0 && rot_dims >= 0 && rot_dims <= D &&
                   rot_dims % 2 == 0 && (rot_dims == 0 || freq_hi) && (!vfreq_hi || E % 2 == 0) &&
                   (pairing == 0 || pairing == 1),
               "b200_headnorm_rot_write: head size %d / %d, rotated %d, pairing %d", D, E, rot_dims,
               pairing);
  const size_t smem = sizeof(float) * (rot_dims + (vfreq_hi ? E : 0) + H + G + 1);
  B200_REQUIRE(smem <= 48 * 1024, "b200_headnorm_rot_write: too many heads");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("headnorm_rot_write", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(headnorm_rot_write_kernel<TT>, dim3(T), dim3(kPoolPrepThreads), smem, st, 1, 0,     \
                static_cast<const TT*>(q), ldq, static_cast<const TT*>(k), ldk,                      \
                static_cast<const TT*>(v), ldv, qw, kw, eps, freq_hi, freq_lo, rot_dims, vfreq_hi,   \
                vfreq_lo, pairing, head_scale, tok_pos, loc, static_cast<TT*>(pool), ld_pool, k_off, \
                v_off, q_out, ldqo, static_cast<TT*>(q_out16), ldqo16, H, G, D, E)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_headnorm_rot_write: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("headnorm_rot_write_kernel");
  return 0;
}

extern "C" int b200_pool_block_means(const void* pool, int64_t ld_pool, int width, float* pooled,
                                     int64_t ld_pooled, int P, int pdiv, const int* req_to_token,
                                     int64_t ld_r2t, const int64_t* req_idx, const int* tok_pos,
                                     const int* tok_b, int T, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(pool && pooled && req_to_token && req_idx && tok_pos && tok_b, "b200_pool_block_means: null pointer");
  B200_REQUIRE(T > 0 && width > 0 && P > 0 && (pdiv == 1 || pdiv == P) && ld_pooled >= width,
               "b200_pool_block_means: width %d, block %d, divisor %d", width, P, pdiv);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("pool_block_means", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(pool_block_means_kernel<TT>, dim3(T), dim3(128), 0, st, 1, 0,                       \
                static_cast<const TT*>(pool), ld_pool, width, pooled, ld_pooled, P, pdiv,            \
                req_to_token, ld_r2t, req_idx, tok_pos, tok_b)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_pool_block_means: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("pool_block_means_kernel");
  return 0;
}

static int pooled_window_attn_impl(const float* q, int64_t ldq, const void* pool, int64_t ld_pool,
                                   int k_off, int v_off, const float* pooled, int64_t ld_pooled, int P,
                                   int pdiv, const int* req_to_token, int64_t ld_r2t,
                                   const int64_t* req_idx, const int* tok_pos, const int* tok_b,
                                   float scale, int window, const float* vfreq_hi, const float* vfreq_lo,
                                   int pairing, void* out, int64_t ldo, int T, int H, int G, int D, int E,
                                   const int* tok_list, int max_keys, float* part_out, int64_t ld_part,
                                   float* part_lse, int64_t ld_lse, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(q && pool && req_to_token && req_idx && tok_pos && tok_b && (out || part_out),
               "b200_pooled_window_attn: null pointer");
  B200_REQUIRE(!part_out || (part_lse && pooled && ld_part >= static_cast<int64_t>(H) * E && ld_lse >= H),
               "b200_pooled_window_attn: the block part needs its buffers and a summary");
  B200_REQUIRE(T > 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && E > 0 && E <= 32 * kPwMaxCols &&
                   window >= 0 && G <= 65535 && (!pooled || (P > 0 && window > 0 && (pdiv == 1 || pdiv == P))) &&
                   (!vfreq_hi || E % 2 == 0),
               "b200_pooled_window_attn: heads %d / %d, key size %d, value size %d (max %d), block %d", H,
               G, D, E, 32 * kPwMaxCols, P);
  // one warp per 64 keys of the longest list (a hint; 0 = unknown), at least 4; the block part has few
  // keys per row and many rows: one warp per 32 blocks
  int nw = part_out ? min(kPwMaxWarps, max(1, ceil_div(max(max_keys, 1), 32)))
                    : (max_keys <= 0 ? 4 : min(kPwMaxWarps, max(4, ceil_div(max_keys, 64))));
  auto smem_for = [&](int w) {
    return sizeof(float) * (static_cast<size_t>(kPwHeads) * D + static_cast<size_t>(w) * kPwHeads * (E + 3) +
                            kPwHeads + static_cast<size_t>(kPwHeads) * E + E + 4);
  };
  while (nw > 1 && smem_for(nw) > 48 * 1024) nw >>= 1;
  const size_t smem = smem_for(nw);
  B200_REQUIRE(smem <= 48 * 1024, "b200_pooled_window_attn: key size %d too large", D);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("pooled_window_attn", st);
  const dim3 grid(T, G);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(pooled_window_attn_kernel<TT, TT>, grid, dim3(nw * 32), smem, st, 1, 0, q, ldq,      \
                static_cast<const TT*>(pool), ld_pool, k_off, v_off, pooled, ld_pooled, P, pdiv,     \
                req_to_token, ld_r2t, req_idx, tok_pos, tok_b, scale, window, vfreq_hi, vfreq_lo,    \
                pairing, static_cast<TT*>(out), ldo, H, G, D, E, tok_list, part_out, ld_part, part_lse,   \
                ld_lse)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_pooled_window_attn: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("pooled_window_attn_kernel");
  return 0;
}

extern "C" int b200_pooled_window_attn(const float* q, int64_t ldq, const void* pool, int64_t ld_pool,
                                       int k_off, int v_off, const float* pooled, int64_t ld_pooled,
                                       int P, int pdiv, const int* req_to_token, int64_t ld_r2t,
                                       const int64_t* req_idx, const int* tok_pos, const int* tok_b,
                                       float scale, int window, const float* vfreq_hi,
                                       const float* vfreq_lo, int pairing, void* out, int64_t ldo, int T,
                                       int H, int G, int D, int E, const int* tok_list, int max_keys,
                                       int dtype, void* stream) {
  return pooled_window_attn_impl(q, ldq, pool, ld_pool, k_off, v_off, pooled, ld_pooled, P, pdiv,
                                 req_to_token, ld_r2t, req_idx, tok_pos, tok_b, scale, window, vfreq_hi,
                                 vfreq_lo, pairing, out, ldo, T, H, G, D, E, tok_list, max_keys, nullptr, 0,
                                 nullptr, 0, dtype, stream);
}

extern "C" int b200_pooled_blocks_attn_part(const float* q, int64_t ldq, const void* pool, int64_t ld_pool,
                                            int k_off, int v_off, const float* pooled, int64_t ld_pooled,
                                            int P, int pdiv, const int* req_to_token, int64_t ld_r2t,
                                            const int64_t* req_idx, const int* tok_pos, const int* tok_b,
                                            float scale, int window, float* part_out, int64_t ld_part,
                                            float* part_lse, int64_t ld_lse, int T, int H, int G, int D,
                                            int E, const int* tok_list, int max_keys, int dtype,
                                            void* stream) {
  return pooled_window_attn_impl(q, ldq, pool, ld_pool, k_off, v_off, pooled, ld_pooled, P, pdiv,
                                 req_to_token, ld_r2t, req_idx, tok_pos, tok_b, scale, window, nullptr,
                                 nullptr, 0, nullptr, 0, T, H, G, D, E, tok_list, max_keys, part_out,
                                 ld_part, part_lse, ld_lse, dtype, stream);
}

extern "C" int b200_pooled_merge_unrotate(void* out, int64_t ldo, const float* lse1, int64_t ld1,
                                          const float* part, int64_t ld_part, const float* lse2,
                                          int64_t ld2, const float* vfreq_hi, const float* vfreq_lo,
                                          int pairing, const int* tok_pos, const int* tok_list, int T,
                                          int H, int E, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(out && tok_pos && T > 0 && H > 0 && E > 0 && (!part || (lse1 && lse2)) &&
                   (!vfreq_hi || E % 2 == 0) && (pairing == 0 || pairing == 1),
               "b200_pooled_merge_unrotate: bad arguments");
  const size_t smem = sizeof(float) * (static_cast<size_t>(H) * E + E + 2);
  B200_REQUIRE(smem <= 48 * 1024, "b200_pooled_merge_unrotate: %d heads of %d values", H, E);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("pooled_merge_unrotate", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(pooled_merge_unrotate_kernel<TT>, dim3(T), dim3(256), smem, st, 1, 0,               \
                static_cast<TT*>(out), ldo, lse1, ld1, part, ld_part, lse2, ld2, vfreq_hi, vfreq_lo, \
                pairing, tok_pos, tok_list, H, E)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else B200_REQUIRE(false, "b200_pooled_merge_unrotate: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("pooled_merge_unrotate_kernel");
  return 0;
}
