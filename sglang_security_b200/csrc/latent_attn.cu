// Latent (compressed-KV) attention over the paged token pool, in the absorbed form: the pool keeps,
// per token, ONE row [c (R latent coordinates) | kr (rot rotated key coordinates)] shared by all
// heads; a head's unrotated query is folded through its key up-projection beforehand (q_lat = W_uk^T
// q), so the score of key j is (q_lat . c_j + q_rot . kr_j) * scale and the head's output is the
// latent mix sum_j p_j c_j, which the caller expands through the value up-projection.  The same
// kernel serves prompt portions and single decoded tokens: one CTA per (token, group of heads), its
// warps split the visible keys (a causal sliding window of `window` tokens, or everything before
// the token when window <= 0), each with an online softmax, merged through shared memory at the end.
// Scores, softmax weights, angles and all accumulation are fp32 whatever the storage type.
//
//   latent_prep : the step before it.  RMS norm (fp32, vector weight) of the query latent, RMS norm of
//                 the KV latent and interleaved rotary embedding of the shared key part, written
//                 straight into the token's pool row.
#include "common.cuh"
#include "latent_attn_mma.cuh"

#include <cstdlib>

namespace b200 {

constexpr int kPrepThreads = 128;

__device__ __forceinline__ float block_sum128(float v, float* red) {
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

// (u, v) at position p, pair i -> (u cos a - v sin a, v cos a + u sin a), a = p * inv_freq[i], fp32
__device__ __forceinline__ void rotate_pair(float& u, float& v, int pos, float f) {
  float s, c;
  sincosf(static_cast<float>(pos) * f, &s, &c);
  const float u2 = u * c - v * s, v2 = v * c + u * s;
  u = u2;
  v = v2;
}

template <typename T>
__global__ void __launch_bounds__(kPrepThreads)
latent_prep_kernel(const T* __restrict__ qraw, int64_t ldq, int QR, const float* __restrict__ wq,
                   T* __restrict__ cq, int64_t ldcq, const T* __restrict__ kvraw, int64_t ldkv, int R,
                   int rot, int rot_dims, const float* __restrict__ wkv,
                   const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                   const int64_t* __restrict__ loc, T* __restrict__ cache, int64_t ldc, float eps,
                   float rot_scale) {
  __shared__ float red[kPrepThreads / 32];
  const int t = blockIdx.x;
  if (qraw) {
    const T* row = qraw + t * ldq;
    float s = 0.f;
    for (int d = threadIdx.x; d < QR; d += kPrepThreads) {
      const float v = to_float<T>(row[d]);
      s = fmaf(v, v, s);
    }
    const float r = 1.0f / sqrtf(block_sum128(s, red) / static_cast<float>(QR) + eps);
    for (int d = threadIdx.x; d < QR; d += kPrepThreads)
      cq[t * ldcq + d] = from_float<T>(to_float<T>(row[d]) * r * wq[d]);
  }
  if (kvraw) {
    const T* row = kvraw + t * ldkv;
    T* dst = cache + loc[t] * ldc;
    float s = 0.f;
    for (int d = threadIdx.x; d < R; d += kPrepThreads) {
      const float v = to_float<T>(row[d]);
      s = fmaf(v, v, s);
    }
    const float r = 1.0f / sqrtf(block_sum128(s, red) / static_cast<float>(R) + eps);
    for (int d = threadIdx.x; d < R; d += kPrepThreads)
      dst[d] = from_float<T>(to_float<T>(row[d]) * r * wkv[d]);
    const int pos = tok_pos[t];
    for (int i = threadIdx.x; 2 * i < rot; i += kPrepThreads) {
      float u = to_float<T>(row[R + 2 * i]);
      if (2 * i + 1 < rot) {
        float v = to_float<T>(row[R + 2 * i + 1]);
        if (2 * i + 1 < rot_dims) {
          rotate_pair(u, v, pos, inv_freq[i]);
          u *= rot_scale;
          v *= rot_scale;
        }
        dst[R + 2 * i + 1] = from_float<T>(v);
      }
      dst[R + 2 * i] = from_float<T>(u);
    }
  }
}

// HB heads per CTA (their q rows interleaved in shared memory so one vector load feeds HB FMAs),
// RC = ceil(R / 32) output coordinates per lane.
template <typename T, int HB, int RC>
__global__ void __launch_bounds__(256)
latent_attn_kernel(const float* __restrict__ q_lat, int64_t ldql_t, int64_t ldql_h,
                   const T* __restrict__ q_raw, int64_t ldqr_t, int64_t ldqr_h, int q_rot_off,
                   const T* __restrict__ cache, int64_t ldc, const int* __restrict__ r2t,
                   int64_t ld_r2t, const int64_t* __restrict__ req_pool, const int* __restrict__ tok_pos,
                   const int* __restrict__ tok_b, const float* __restrict__ inv_freq, int rot_dims,
                   int H, int R, int rot, int window, float scale, T* __restrict__ out,
                   int64_t ldo_t, int64_t ldo_h) {
  extern __shared__ __align__(16) float smem[];
  const int D = R + rot, Dp = D | 1;
  const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* q_s = smem;                                     // [D][HB]
  float* k_s = q_s + ((D * HB + 3) & ~3) + warp * (32 * Dp + 32 * HB);   // [32][Dp]
  float* p_s = k_s + 32 * Dp;                            // [32][HB]
  const int t = blockIdx.x, h0 = blockIdx.y * HB;
  const int pos = tok_pos[t];
  const int64_t rp = req_pool[tok_b[t]];

  for (int e = threadIdx.x; e < R * HB; e += blockDim.x) {
    const int hh = e / R, d = e - hh * R;
    q_s[d * HB + hh] = (h0 + hh < H) ? q_lat[t * ldql_t + (h0 + hh) * ldql_h + d] : 0.f;
  }
  for (int e = threadIdx.x; e < ((rot + 1) / 2) * HB; e += blockDim.x) {
    const int hh = e / ((rot + 1) / 2), i = e - hh * ((rot + 1) / 2);
    float u = 0.f, v = 0.f;
    if (h0 + hh < H) {
      const T* qr = q_raw + t * ldqr_t + (h0 + hh) * ldqr_h + q_rot_off;
      u = to_float<T>(qr[2 * i]);
      if (2 * i + 1 < rot) v = to_float<T>(qr[2 * i + 1]);
      if (2 * i + 1 < rot_dims) rotate_pair(u, v, pos, inv_freq[i]);
    }
    q_s[(R + 2 * i) * HB + hh] = u;
    if (2 * i + 1 < rot) q_s[(R + 2 * i + 1) * HB + hh] = v;
  }
  __syncthreads();

  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int n = pos - lo + 1;
  const int tiles = (n + 31) >> 5;
  float m[HB], l[HB], acc[HB][RC];
#pragma unroll
  for (int hh = 0; hh < HB; ++hh) {
    m[hh] = -INFINITY;
    l[hh] = 0.f;
#pragma unroll
    for (int i = 0; i < RC; ++i) acc[hh][i] = 0.f;
  }
  for (int tile = warp; tile < tiles; tile += nw) {
    const int j = lo + tile * 32 + lane;
    const bool valid = j <= pos;
    const int64_t slot = valid ? static_cast<int64_t>(r2t[rp * ld_r2t + j]) : 0;
    const int nkeys = min(32, n - tile * 32);
    for (int jj = 0; jj < nkeys; ++jj) {
      const T* row = cache + __shfl_sync(0xffffffffu, slot, jj) * ldc;
      for (int d = lane; d < D; d += 32) k_s[jj * Dp + d] = to_float<T>(row[d]);
    }
    __syncwarp();
    float s[HB];
#pragma unroll
    for (int hh = 0; hh < HB; ++hh) s[hh] = 0.f;
    if (valid) {
      const float* kr = k_s + lane * Dp;
      for (int d = 0; d < D; ++d) {
        const float kv = kr[d];
#pragma unroll
        for (int hh = 0; hh < HB; ++hh) s[hh] = fmaf(kv, q_s[d * HB + hh], s[hh]);
      }
    }
#pragma unroll
    for (int hh = 0; hh < HB; ++hh) {
      const float sc = valid ? s[hh] * scale : -INFINITY;
      float mx = sc;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float mn = fmaxf(m[hh], mx);
      const float p = valid ? expf(sc - mn) : 0.f;
      float ps = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ps += __shfl_xor_sync(0xffffffffu, ps, o);
      const float corr = expf(m[hh] - mn);   // 0 on the first tile (m = -inf)
      l[hh] = l[hh] * corr + ps;
      m[hh] = mn;
#pragma unroll
      for (int i = 0; i < RC; ++i) acc[hh][i] *= corr;
      p_s[lane * HB + hh] = p;
    }
    __syncwarp();
    for (int jj = 0; jj < nkeys; ++jj) {
      float p[HB];
#pragma unroll
      for (int hh = 0; hh < HB; ++hh) p[hh] = p_s[jj * HB + hh];
#pragma unroll
      for (int i = 0; i < RC; ++i) {
        const int d = lane + 32 * i;
        const float cv = d < R ? k_s[jj * Dp + d] : 0.f;
#pragma unroll
        for (int hh = 0; hh < HB; ++hh) acc[hh][i] = fmaf(p[hh], cv, acc[hh][i]);
      }
    }
    __syncwarp();
  }
  // merge the warps' partial softmaxes: each warp leaves [HB][R + 2] = (m, l, acc) in its own tile area
  float* mine = k_s;
#pragma unroll
  for (int hh = 0; hh < HB; ++hh) {
    if (lane == 0) {
      mine[hh * (R + 2)] = m[hh];
      mine[hh * (R + 2) + 1] = l[hh];
    }
#pragma unroll
    for (int i = 0; i < RC; ++i) {
      const int d = lane + 32 * i;
      if (d < R) mine[hh * (R + 2) + 2 + d] = acc[hh][i];
    }
  }
  __syncthreads();
  const float* base = q_s + ((D * HB + 3) & ~3);
  const int wstride = 32 * Dp + 32 * HB;
  for (int e = threadIdx.x; e < HB * R; e += blockDim.x) {
    const int hh = e / R, d = e - hh * R;
    if (h0 + hh >= H) continue;
    float M = -INFINITY;
    for (int w = 0; w < nw; ++w) M = fmaxf(M, base[w * wstride + hh * (R + 2)]);
    float L = 0.f, o = 0.f;
    for (int w = 0; w < nw; ++w) {
      const float* pw = base + w * wstride + hh * (R + 2);
      if (pw[0] == -INFINITY) continue;
      const float f = expf(pw[0] - M);
      L = fmaf(pw[1], f, L);
      o = fmaf(pw[2 + d], f, o);
    }
    out[t * ldo_t + (h0 + hh) * ldo_h + d] = from_float<T>(o / L);
  }
}

template <typename T, int HB, int RC>
static int latent_attn_launch(dim3 grid, int nw, size_t smem, cudaStream_t st, const float* q_lat,
                              int64_t ldql_t, int64_t ldql_h, const void* q_raw, int64_t ldqr_t,
                              int64_t ldqr_h, int q_rot_off, const void* cache, int64_t ldc,
                              const int* r2t, int64_t ld_r2t, const int64_t* req_pool,
                              const int* tok_pos, const int* tok_b, const float* inv_freq, int rot_dims,
                              int H, int R, int rot, int window, float scale, void* out, int64_t ldo_t,
                              int64_t ldo_h) {
  auto kern = latent_attn_kernel<T, HB, RC>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
  launch_kernel(kern, grid, dim3(nw * 32), smem, st, 1, 0, q_lat, ldql_t, ldql_h,
                static_cast<const T*>(q_raw), ldqr_t, ldqr_h, q_rot_off, static_cast<const T*>(cache),
                ldc, r2t, ld_r2t, req_pool, tok_pos, tok_b, inv_freq, rot_dims, H, R, rot, window,
                scale, static_cast<T*>(out), ldo_t, ldo_h);
  B200_CHECK_LAUNCH("latent_attn_kernel");
  note_variant("latent_attn hb%d rc%d warps%d smem%zu", HB, RC, nw, smem);
  return 0;
}

template <typename T>
static int latent_attn_dispatch(int T_tokens, int max_keys, cudaStream_t st, const float* q_lat,
                                int64_t ldql_t, int64_t ldql_h, const void* q_raw, int64_t ldqr_t,
                                int64_t ldqr_h, int q_rot_off, const void* cache, int64_t ldc,
                                const int* r2t, int64_t ld_r2t, const int64_t* req_pool,
                                const int* tok_pos, const int* tok_b, const float* inv_freq,
                                int rot_dims, int H, int R, int rot, int window, float scale, void* out,
                                int64_t ldo_t, int64_t ldo_h) {
  const int rc = ceil_div(R, 32);
  B200_REQUIRE(rc <= 16, "b200_latent_attn: latent size %d above 512", R);
  // heads per CTA: as many as the accumulators allow (HB * RC <= 64 registers), no more than needed
  int hb = rc <= 8 ? 8 : 4;
  while (hb > 1 && hb / 2 >= H) hb /= 2;
  const int D = R + rot, Dp = D | 1;
  const size_t per_warp = static_cast<size_t>(32 * Dp + 32 * hb) * 4;
  const size_t fixed = static_cast<size_t>((D * hb + 3) & ~3) * 4;
  int nw = min(8, max(1, ceil_div(max_keys, 32)));
  while (nw > 1 && fixed + nw * per_warp > 200 * 1024) --nw;
  B200_REQUIRE(fixed + nw * per_warp <= 227 * 1024, "b200_latent_attn: rows of %d do not fit", D);
  const size_t smem = fixed + nw * per_warp;
  const dim3 grid(T_tokens, ceil_div(H, hb));
#define GO(HB, RC)                                                                                   \
  return latent_attn_launch<T, HB, RC>(grid, nw, smem, st, q_lat, ldql_t, ldql_h, q_raw, ldqr_t,     \
                                       ldqr_h, q_rot_off, cache, ldc, r2t, ld_r2t, req_pool, tok_pos, \
                                       tok_b, inv_freq, rot_dims, H, R, rot, window, scale, out,      \
                                       ldo_t, ldo_h)
#define BY_RC(HB)                                                                                    \
  do {                                                                                               \
    if (rc <= 1) GO(HB, 1);                                                                          \
    if (rc <= 2) GO(HB, 2);                                                                          \
    if (rc <= 4) GO(HB, 4);                                                                          \
    GO(HB, 8);                                                                                       \
  } while (0)
  if (rc > 8) {
    if (hb == 4) GO(4, 16);
    if (hb == 2) GO(2, 16);
    GO(1, 16);
  }
  if (hb == 8) BY_RC(8);
  if (hb == 4) BY_RC(4);
  if (hb == 2) BY_RC(2);
  BY_RC(1);
#undef BY_RC
#undef GO
}

template <typename T, int CW>
static int latent_attn_mma_launch(int grid_x, int grid_y, size_t smem, cudaStream_t st, const float* q_lat,
                                  int64_t ldql_t, int64_t ldql_h, const void* q_raw, int64_t ldqr_t,
                                  int64_t ldqr_h, int q_rot_off, const void* cache, int64_t ldc,
                                  const int* r2t, int64_t ld_r2t, const int64_t* req_pool,
                                  const int* tok_pos, const int* ext_start, const int* ext_len, int bs,
                                  const float* inv_freq, int rot_dims, int H, int HG, int TQ, int R,
                                  int rot, int window, float scale, void* out, int64_t ldo_t,
                                  int64_t ldo_h, int nsplit, float* ws) {
  auto kern = latent_attn_mma_kernel<T, CW>;
  if (smem > 48 * 1024)
    B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(smem)));
  launch_kernel(kern, dim3(grid_x, grid_y, nsplit), dim3(kLaThreads), smem, st, 1, 0, q_lat, ldql_t, ldql_h,
                static_cast<const T*>(q_raw), ldqr_t, ldqr_h, q_rot_off, static_cast<const T*>(cache),
                ldc, r2t, ld_r2t, req_pool, tok_pos, ext_start, ext_len, bs, inv_freq, rot_dims, H, HG,
                TQ, R, rot, window, scale, static_cast<T*>(out), ldo_t, ldo_h, nsplit, ws, grid_x);
  B200_CHECK_LAUNCH("latent_attn_mma_kernel");
  if (nsplit > 1) {
    launch_kernel(latent_attn_merge_kernel<T>, dim3(grid_x * H), dim3(128), 0, st, 1, 0,
                  static_cast<const float*>(ws), nsplit, grid_x, H, R, static_cast<T*>(out), ldo_t, ldo_h);
    B200_CHECK_LAUNCH("latent_attn_merge_kernel");
  }
  note_variant("latent_attn_mma cw%d hg%d tq%d smem%zu splits%d", CW, HG, TQ, smem, nsplit);
  return 0;
}

// ---- expanded (per-head) keys and values for long prompt portions -------------------------------
// A portion of a prompt whose tokens outnumber the keys it has to expand is cheaper as ordinary
// multi-head attention over K_h = [W_uk_h c | kr] and V_h = W_uv_h c (head size D) than over the
// latent itself (head size R + rot): the two kernels below stage its operands around one GEMM.
//   blocks [0, N):      c_out[n, :R]  = cache[slots[n], :R]             (A operand of the up-projection)
//   blocks [N, N + T):  q_out[t, h, :] = [q[t, h, :dim] | rotary(q[t, h, dim:dim+rot]) | 0...]   (D wide)
template <typename T>
__global__ void __launch_bounds__(256)
latent_expand_gather_kernel(const T* __restrict__ cache, int64_t ldc, const int64_t* __restrict__ slots,
                            int N, int R, T* __restrict__ c_out, int64_t ldco, const T* __restrict__ q,
                            int64_t ldq_t, int64_t ldq_h, int H, int dim, int rot, int rot_dims,
                            const float* __restrict__ inv_freq, const int* __restrict__ tok_pos,
                            T* __restrict__ q_out, int D) {
  const int blk = blockIdx.x;
  if (blk < N) {
    const T* src = cache + slots[blk] * ldc;
    T* dst = c_out + blk * ldco;
    for (int d = threadIdx.x; d < R; d += blockDim.x) dst[d] = src[d];
    return;
  }
  const int t = blk - N;
  const float pos = static_cast<float>(tok_pos[t]);
  const int dq = dim + rot;
  for (int e = threadIdx.x; e < H * D; e += blockDim.x) {
    const int h = e / D, d = e - h * D;
    const T* qh = q + t * ldq_t + h * ldq_h;
    float v = 0.f;
    if (d < dim) {
      v = to_float<T>(qh[d]);
    } else if (d < dq) {
      const int r = d - dim;
      v = to_float<T>(qh[d]);
      if ((r | 1) < rot_dims) {                        // pair (2i, 2i + 1) inside the rotated dims
        const float other = to_float<T>(qh[dim + (r ^ 1)]);
        float sn, cs;
        sincosf(pos * inv_freq[r >> 1], &sn, &cs);
        v = (r & 1) ? v * cs + other * sn : v * cs - other * sn;
      }
    }
    q_out[(static_cast<int64_t>(t) * H + h) * D + d] = from_float<T>(v);
  }
}

// kv[n, h, dim + i] = cache[slots[n], R + i] for every head: the rotated key part, shared by all heads
template <typename T>
__global__ void __launch_bounds__(256)
latent_expand_rotkeys_kernel(const T* __restrict__ cache, int64_t ldc, const int64_t* __restrict__ slots,
                             int R, int rot, T* __restrict__ k_out, int64_t ldk, int H, int D, int dim) {
  const T* src = cache + slots[blockIdx.x] * ldc + R;
  T* dst = k_out + blockIdx.x * ldk + dim;
  for (int e = threadIdx.x; e < H * rot; e += blockDim.x) {
    const int h = e / rot, i = e - h * rot;
    dst[h * D + i] = src[i];
  }
}

static bool latent_attn_mma_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("B200_LATENT_ATTN_MMA");
    return !(e && e[0] == '0');
  }();
  return on;
}

}  // namespace b200

extern "C" int b200_latent_prep_scaled(const void* qraw, int64_t ldq, int QR, const float* wq, void* cq,
                                int64_t ldcq, const void* kvraw, int64_t ldkv, int R, int rot,
                                int rot_dims, const float* wkv, const float* inv_freq,
                                const int* tok_pos, const int64_t* loc, void* cache, int64_t ldc,
                                float eps, float rot_scale, int T, int dtype,
                                       void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(qraw || kvraw, "b200_latent_prep: nothing to do");
  B200_REQUIRE(!qraw || (wq && cq && QR > 0), "b200_latent_prep: query latent arguments");
  B200_REQUIRE(!kvraw || (wkv && tok_pos && loc && cache && R > 0 && rot >= 0 && rot_dims <= rot &&
                          rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq)),
               "b200_latent_prep: KV latent arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("latent_prep", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(latent_prep_kernel<TT>, dim3(T), dim3(kPrepThreads), 0, st, 1, 0,                    \
                static_cast<const TT*>(qraw), ldq, QR, wq, static_cast<TT*>(cq), ldcq,               \
                static_cast<const TT*>(kvraw), ldkv, R, rot, rot_dims, wkv, inv_freq, tok_pos, loc,  \
                static_cast<TT*>(cache), ldc, eps, rot_scale)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_latent_prep: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("latent_prep_kernel");
  return 0;
}

extern "C" int b200_latent_prep(const void* qraw, int64_t ldq, int QR, const float* wq, void* cq,
                                int64_t ldcq, const void* kvraw, int64_t ldkv, int R, int rot,
                                int rot_dims, const float* wkv, const float* inv_freq,
                                const int* tok_pos, const int64_t* loc, void* cache, int64_t ldc,
                                float eps, int T, int dtype, void* stream) {
  return b200_latent_prep_scaled(qraw, ldq, QR, wq, cq, ldcq, kvraw, ldkv, R, rot, rot_dims, wkv,
                                 inv_freq, tok_pos, loc, cache, ldc, eps, 1.0f, T, dtype, stream);
}

extern "C" int b200_latent_attn(const float* q_lat, int64_t ldql_t, int64_t ldql_h, const void* q_raw,
                                int64_t ldqr_t, int64_t ldqr_h, int q_rot_off, const void* cache,
                                int64_t ldc, const int* r2t, int64_t ld_r2t, const int64_t* req_pool,
                                const int* tok_pos, const int* tok_b, const int* ext_start,
                                const int* ext_len, int bs, const float* inv_freq, int rot_dims, int T,
                                int H, int R, int rot, int window, int max_keys, float scale, void* out,
                                int64_t ldo_t, int64_t ldo_h, int num_splits, float* ws,
                                int64_t ws_floats, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(q_lat && cache && r2t && req_pool && tok_pos && tok_b && out,
               "b200_latent_attn: null pointer");
  B200_REQUIRE(H > 0 && R > 0 && rot >= 0 && (rot == 0 || q_raw) && rot_dims <= rot &&
                   rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq),
               "b200_latent_attn: bad sizes (H %d R %d rot %d rot_dims %d)", H, R, rot, rot_dims);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("latent_attn", st);
  if (max_keys <= 0) max_keys = 1 << 30;
  if (window > 0) max_keys = min(max_keys, window);
  // 16-bit storage with 16-byte-copyable rows: the tensor-core instance
  const int R16 = (R + 15) & ~15, rot16 = (rot + 15) & ~15;
  if ((dtype == B200_BF16 || dtype == B200_F16) && latent_attn_mma_enabled() && ext_start && ext_len &&
      bs > 0 && R % 8 == 0 && rot % 8 == 0 && ldc % 8 == 0 && aligned16(cache) && R16 <= 512) {
    const int HG = min(H, kLaRows), TQ = kLaRows / HG;
    const size_t smem = static_cast<size_t>(kLaRows + 2 * kLaKeys) * (R16 + rot16 + 8) * 2;
    const int gy = ceil_div(H, HG);
    int nsplit = max(1, num_splits);
    if (nsplit > 1)
      B200_REQUIRE(ws && ws_floats >= static_cast<int64_t>(nsplit) * T * H * (R + 2),
                   "b200_latent_attn: workspace too small for %d splits", nsplit);
#define GO_MMA(TT, CW)                                                                               \
  return latent_attn_mma_launch<TT, CW>(T, gy, smem, st, q_lat, ldql_t, ldql_h, q_raw, ldqr_t, ldqr_h, \
                                        q_rot_off, cache, ldc, r2t, ld_r2t, req_pool, tok_pos,        \
                                        ext_start, ext_len, bs, inv_freq, rot_dims, H, HG, TQ, R, rot, \
                                        window, scale, out, ldo_t, ldo_h, nsplit, ws)
#define BY_CW(TT)                      \
  do {                                 \
    if (R16 <= 32) GO_MMA(TT, 16);     \
    if (R16 <= 64) GO_MMA(TT, 32);     \
    if (R16 <= 128) GO_MMA(TT, 64);    \
    if (R16 <= 256) GO_MMA(TT, 128);   \
    GO_MMA(TT, 256);                   \
  } while (0)
    if (dtype == B200_BF16) BY_CW(__nv_bfloat16);
    BY_CW(__half);
#undef BY_CW
#undef GO_MMA
  }
#define GO(TT)                                                                                       \
  return latent_attn_dispatch<TT>(T, max_keys, st, q_lat, ldql_t, ldql_h, q_raw, ldqr_t, ldqr_h,     \
                                  q_rot_off, cache, ldc, r2t, ld_r2t, req_pool, tok_pos, tok_b,      \
                                  inv_freq, rot_dims, H, R, rot, window, scale, out, ldo_t, ldo_h)
  if (dtype == B200_BF16) GO(__nv_bfloat16);
  if (dtype == B200_F16) GO(__half);
  if (dtype == B200_F32) GO(float);
#undef GO
  B200_REQUIRE(false, "b200_latent_attn: dtype %d", dtype);
}

extern "C" int b200_latent_expand_gather(const void* cache, int64_t ldc, const int64_t* slots, int N,
                                         int R, void* c_out, int64_t ldco, const void* q,
                                         int64_t ldq_t, int64_t ldq_h, int H, int dim, int rot,
                                         int rot_dims, const float* inv_freq, const int* tok_pos,
                                         void* q_out, int D, int T, int dtype, void* stream) {
  using namespace b200;
  if (N + T == 0) return 0;
  B200_REQUIRE(cache && slots && c_out && q && tok_pos && q_out, "b200_latent_expand_gather: null pointer");
  B200_REQUIRE(N >= 0 && T >= 0 && R > 0 && H > 0 && dim >= 0 && rot >= 0 && dim + rot <= D &&
                   rot_dims <= rot && rot_dims % 2 == 0 && (rot_dims == 0 || inv_freq),
               "b200_latent_expand_gather: bad sizes (dim %d rot %d D %d rot_dims %d)", dim, rot, D, rot_dims);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("latent_expand", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(latent_expand_gather_kernel<TT>, dim3(N + T), dim3(256), 0, st, 1, 0,                \
                static_cast<const TT*>(cache), ldc, slots, N, R, static_cast<TT*>(c_out), ldco,      \
                static_cast<const TT*>(q), ldq_t, ldq_h, H, dim, rot, rot_dims, inv_freq, tok_pos,   \
                static_cast<TT*>(q_out), D)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else B200_REQUIRE(false, "b200_latent_expand_gather: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("latent_expand_gather_kernel");
  return 0;
}

extern "C" int b200_latent_expand_rotkeys(const void* cache, int64_t ldc, const int64_t* slots, int N,
                                          int R, int rot, void* k_out, int64_t ldk, int H, int D,
                                          int dim, int dtype, void* stream) {
  using namespace b200;
  if (N == 0 || rot == 0) return 0;
  B200_REQUIRE(cache && slots && k_out && H > 0 && dim >= 0 && dim + rot <= D,
               "b200_latent_expand_rotkeys: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("latent_expand", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(latent_expand_rotkeys_kernel<TT>, dim3(N), dim3(256), 0, st, 1, 0,                   \
                static_cast<const TT*>(cache), ldc, slots, R, rot, static_cast<TT*>(k_out), ldk, H,  \
                D, dim)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else B200_REQUIRE(false, "b200_latent_expand_rotkeys: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("latent_expand_rotkeys_kernel");
  return 0;
}
