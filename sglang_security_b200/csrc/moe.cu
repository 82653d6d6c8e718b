// Mixture-of-experts feed-forward, device side only (no host read of the routing result):
//   moe_route        : router logits z = W_r h + b in fp32, the `top` largest (ties: lowest index),
//                      weights = softmax over the chosen logits, or (score mode 1) the sigmoid of each
//                      chosen logit, not renormalised; optionally the per-token gate
//                      sigmoid(w_sg . h) of a shared expert.  One CTA per token.
//   moe_align        : stable counting sort of the (token, choice) rows by expert -> row offsets per
//                      expert and the sorted row list.
//   moe_grouped_gemm : for every expert, rows[offsets[e] : offsets[e+1]] x W[e]^T with fp32
//                      accumulation.  GATED: A rows are gathered from the token activations, both
//                      halves of the fused [gate; up] weight are multiplied in one pass and
//                      act(gate) * up is stored in sorted order; otherwise A is that intermediate and
//                      the result is scattered back to row t * top + k for the weighted combine.
//                      ACT form (experts without a gate): A rows gathered like GATED, one weight,
//                      act(scale[row] * (W h)) stored in sorted order; the optional fp32 scale per
//                      (token, choice) row is a router weight that multiplies the expert's input,
//                      applied to the fp32 accumulator (W (s h) = s (W h)).
#include "common.cuh"
#include "latent_attn_mma.cuh"   // ldmatrix / mma.sync wrappers

namespace b200 {

constexpr int kMaxExpertsPerLane = 8;  // experts <= 256

// Router logits of one token: the CTA's 8 warps share the experts' dot products (and the optional
// shared-expert gate's); z_s[e] = w_e . h + b_e in fp32.
template <typename T>
__device__ __forceinline__ void route_logits(const T* __restrict__ h, int64_t ldh,
                                             const float* __restrict__ wr, const float* __restrict__ br,
                                             int E, int W, const float* __restrict__ wsg,
                                             float* __restrict__ gate, int t, float* z_s) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const T* row = h + t * ldh;
  const int jobs = E + ((wsg && gate) ? 1 : 0);
  // every token takes the same path, so its sums do not depend on the batch it arrives in
  const bool vec8 = W % 8 == 0 && ldh % 8 == 0 && (reinterpret_cast<uintptr_t>(h) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(wr) & 15) == 0 &&
                    (!wsg || (reinterpret_cast<uintptr_t>(wsg) & 15) == 0);
  for (int e = warp; e < jobs; e += 8) {
    const float* w = e < E ? wr + static_cast<int64_t>(e) * W : wsg;
    float s0 = 0.f, s1 = 0.f;
    if (vec8) {
      // a lane takes 8 consecutive coordinates per pass: one 16-byte load of the activations
      // (two for fp32) against two of the router row
      for (int d = lane * 8; d < W; d += 256) {
        float hv[8];
        if constexpr (sizeof(T) == 2) {
          const uint4 u = *reinterpret_cast<const uint4*>(row + d);
          const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
          for (int k = 0; k < 8; ++k) hv[k] = to_float<T>(e[k]);
        } else {
          const float4 h0 = *reinterpret_cast<const float4*>(row + d);
          const float4 h1 = *reinterpret_cast<const float4*>(row + d + 4);
          hv[0] = h0.x, hv[1] = h0.y, hv[2] = h0.z, hv[3] = h0.w;
          hv[4] = h1.x, hv[5] = h1.y, hv[6] = h1.z, hv[7] = h1.w;
        }
        const float4 w0 = *reinterpret_cast<const float4*>(w + d);
        const float4 w1 = *reinterpret_cast<const float4*>(w + d + 4);
        s0 = fmaf(w0.x, hv[0], s0);
        s1 = fmaf(w1.x, hv[4], s1);
        s0 = fmaf(w0.y, hv[1], s0);
        s1 = fmaf(w1.y, hv[5], s1);
        s0 = fmaf(w0.z, hv[2], s0);
        s1 = fmaf(w1.z, hv[6], s1);
        s0 = fmaf(w0.w, hv[3], s0);
        s1 = fmaf(w1.w, hv[7], s1);
      }
    } else {
      int d = lane;
      for (; d + 32 < W; d += 64) {
        s0 = fmaf(w[d], to_float<T>(row[d]), s0);
        s1 = fmaf(w[d + 32], to_float<T>(row[d + 32]), s1);
      }
      if (d < W) s0 = fmaf(w[d], to_float<T>(row[d]), s0);
    }
    float s = s0 + s1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
      if (e < E) z_s[e] = s + (br ? br[e] : 0.f);
      else gate[t] = 1.0f / (1.0f + expf(-s));
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ h, int64_t ldh, const float* __restrict__ wr,
                 const float* __restrict__ br, int E, int W, int top, const float* __restrict__ wsg,
                 int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ gate, int Tn,
                 int score) {
  // one CTA per token: its 8 warps share the experts' dot products (and the gate's), warp 0 ranks
  __shared__ float z_s[32 * kMaxExpertsPerLane];
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  route_logits<T>(h, ldh, wr, br, E, W, wsg, gate, t, z_s);
  __syncthreads();
  if (warp != 0) return;
  float z[kMaxExpertsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) z[i] = (lane + 32 * i < E) ? z_s[lane + 32 * i] : -INFINITY;
  float zmax = 0.f, sum = 0.f, mine = 0.f, mine_z = 0.f;  // lane k keeps the k-th chosen logit
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < E && (z[i] > bv || (z[i] == bv && e < bi))) {
        bv = z[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (k == 0) zmax = bv;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i)
      if (bi == lane + 32 * i) z[i] = -INFINITY;
    const float p = expf(bv - zmax);
    sum += p;
    if (lane == k) {
      mine = p;
      mine_z = bv;
    }
    if (lane == 0) ids[t * top + k] = bi;
  }
  if (lane < top) wts[t * top + lane] = score == 1 ? 1.0f / (1.0f + expf(-mine_z)) : mine / sum;
}

// Softmax scores over ALL experts, a choice among groups of neighbouring experts:
//   s = softmax(z);  choice = s + correction;  a group's score is its largest choice score; only experts
//   of the `keep` best groups can be chosen (the others count as minus infinity);  the `top` largest choice
//   scores are taken (ties: lowest index);  weights = s of the chosen / (their sum + 1e-20).
template <typename T>
__global__ void __launch_bounds__(256)
moe_route_grouped_kernel(const T* __restrict__ h, int64_t ldh, const float* __restrict__ wr,
                         const float* __restrict__ correction, int E, int W, int top, int n_groups,
                         int keep, int* __restrict__ ids, float* __restrict__ wts) {
  __shared__ float z_s[32 * kMaxExpertsPerLane];   // logits, then the scores s
  __shared__ float c_s[32 * kMaxExpertsPerLane];   // choice scores
  __shared__ float g_s[32 * kMaxExpertsPerLane];   // group scores
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  route_logits<T>(h, ldh, wr, nullptr, E, W, nullptr, nullptr, t, z_s);
  __syncthreads();
  if (warp != 0) return;
  float zmax = -INFINITY;
  for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z_s[e]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) zmax = fmaxf(zmax, __shfl_xor_sync(0xffffffffu, zmax, o));
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(z_s[e] - zmax);
    z_s[e] = p;
    sum += p;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  for (int e = lane; e < E; e += 32) {
    z_s[e] /= sum;
    c_s[e] = z_s[e] + (correction ? correction[e] : 0.f);
  }
  __syncwarp();
  if (n_groups > 1 && keep < n_groups) {
    const int per = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float gm = -INFINITY;
      for (int i = 0; i < per; ++i) gm = fmaxf(gm, c_s[g * per + i]);
      g_s[g] = gm;
    }
    __syncwarp();
    // the `keep` best groups, one per pass (ties: lowest index); a kept group's score becomes +inf
    for (int k = 0; k < keep; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32) {
        const float v = g_s[g];
        if (v != INFINITY && (v > bv || (v == bv && g < bi))) {
          bv = v;
          bi = g;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
          bv = ov;
          bi = oi;
        }
      }
      if (lane == 0 && bi != 0x7fffffff) g_s[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (g_s[e / per] != INFINITY) c_s[e] = -INFINITY;
    __syncwarp();
  }
  float z[kMaxExpertsPerLane];
#pragma unroll
  for (int i = 0; i < kMaxExpertsPerLane; ++i) z[i] = (lane + 32 * i < E) ? c_s[lane + 32 * i] : -INFINITY;
  float wsum = 0.f, mine = 0.f;                 // lane k keeps the k-th chosen expert's score
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i) {
      const int e = lane + 32 * i;
      if (e < E && z[i] != -INFINITY && (z[i] > bv || (z[i] == bv && e < bi))) {
        bv = z[i];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) {
        bv = ov;
        bi = oi;
      }
    }
    if (bi == 0x7fffffff) bi = 0;               // fewer allowed experts than `top` (rejected by the host)
#pragma unroll
    for (int i = 0; i < kMaxExpertsPerLane; ++i)
      if (bi == lane + 32 * i) z[i] = -INFINITY;
    const float sc = z_s[bi];
    wsum += sc;
    if (lane == k) mine = sc;
    if (lane == 0) ids[t * top + k] = bi;
  }
  if (lane < top) wts[t * top + lane] = mine / (wsum + 1e-20f);
}

__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ ids, int N, int E, int* __restrict__ offsets,
                 int* __restrict__ sorted_rows) {
  extern __shared__ int cnt[];  // [E + 1]
  for (int e = threadIdx.x; e <= E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < N; i += blockDim.x) atomicAdd(&cnt[ids[i] + 1], 1);
  __syncthreads();
  if (threadIdx.x == 0)
    for (int e = 0; e < E; ++e) cnt[e + 1] += cnt[e];
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = cnt[e];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int e = warp; e < E; e += nw) {
    int base = cnt[e];
    for (int i0 = 0; i0 < N; i0 += 32) {
      const int i = i0 + lane;
      const bool hit = i < N && ids[i] == e;
      const unsigned mask = __ballot_sync(0xffffffffu, hit);
      if (hit) sorted_rows[base + __popc(mask & ((1u << lane) - 1u))] = i;
      base += __popc(mask);
    }
  }
}

__device__ __forceinline__ float moe_act(float z, int kind) {
  if (kind == 0) return z / (1.0f + expf(-z));
  if (kind == 2) {                                   // squared relu
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  const float u = 0.7978845608028654f * (z + 0.044715f * z * z * z);
  return 0.5f * z * (1.0f + tanhf(u));
}

constexpr int kGM = 32, kGN = 64, kGK = 32;

// MODE 0: plain (A sorted, result scattered); 1: gated; 2: one weight + activation (see the top)
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_grouped_gemm_kernel(const T* __restrict__ a, int64_t lda, const T* __restrict__ w, int64_t ldw,
                        int64_t w_expert_stride, const int* __restrict__ offsets,
                        const int* __restrict__ sorted_rows, int E, int top, int Nout, int K,
                        T* __restrict__ out, int64_t ldo, int act,
                        const float* __restrict__ row_scale) {
  constexpr bool GATED = MODE == 1;
  constexpr bool GATHER = MODE != 0;
  __shared__ float As[kGM][kGK + 1];
  __shared__ float Bs[(GATED ? 2 : 1) * kGN][kGK + 1];
  __shared__ int rows[kGM];
  // which expert and which of its row tiles this CTA has
  int e = 0, tile = blockIdx.x, lo = 0, hi = 0;
  for (; e < E; ++e) {
    lo = offsets[e];
    hi = offsets[e + 1];
    const int nt = (hi - lo + kGM - 1) / kGM;
    if (tile < nt) break;
    tile -= nt;
  }
  if (e >= E) return;
  const int m0 = lo + tile * kGM, mcount = min(kGM, hi - m0);
  const int n0 = blockIdx.y * kGN;
  if (threadIdx.x < kGM) {
    int r = -1;
    if (threadIdx.x < mcount) r = sorted_rows[m0 + threadIdx.x];
    rows[threadIdx.x] = r;
  }
  __syncthreads();
  const T* we = w + e * w_expert_stride;
  const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
  float acc[2][4], acc2[2][4];
#pragma unroll
  for (int r = 0; r < 2; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = acc2[r][c] = 0.f;
  for (int k0 = 0; k0 < K; k0 += kGK) {
    for (int idx = threadIdx.x; idx < kGM * kGK; idx += 256) {
      const int r = idx / kGK, k = idx - r * kGK;
      float v = 0.f;
      if (r < mcount && k0 + k < K) {
        const int64_t src = GATHER ? rows[r] / top : m0 + r;
        v = to_float<T>(a[src * lda + k0 + k]);
      }
      As[r][k] = v;
    }
    for (int idx = threadIdx.x; idx < (GATED ? 2 : 1) * kGN * kGK; idx += 256) {
      const int r = idx / kGK, k = idx - r * kGK;
      const int half = r / kGN, n = n0 + (r - half * kGN);
      float v = 0.f;
      if (n < Nout && k0 + k < K) v = to_float<T>(we[(static_cast<int64_t>(half) * Nout + n) * ldw + k0 + k]);
      Bs[r][k] = v;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < kGK; ++k) {
      const float a0 = As[ty * 2][k], a1 = As[ty * 2 + 1][k];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float b = Bs[tx + 16 * c][k];
        acc[0][c] = fmaf(a0, b, acc[0][c]);
        acc[1][c] = fmaf(a1, b, acc[1][c]);
        if (GATED) {
          const float b2 = Bs[kGN + tx + 16 * c][k];
          acc2[0][c] = fmaf(a0, b2, acc2[0][c]);
          acc2[1][c] = fmaf(a1, b2, acc2[1][c]);
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int lr = ty * 2 + r;
    if (lr >= mcount) continue;
    const int64_t orow = GATHER ? m0 + lr : rows[lr];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int n = n0 + tx + 16 * c;
      if (n >= Nout) continue;
      float v = acc[r][c];
      if (GATED) v = moe_act(v, act) * acc2[r][c];
      else if (MODE == 2) v = moe_act(row_scale ? v * row_scale[rows[lr]] : v, act);
      out[orow * ldo + n] = from_float<T>(v);
    }
  }
}

// Tensor-core instance for 16-bit types (K a multiple of 8, 16-byte aligned rows): TM sorted rows of
// one expert x 64 output columns (gated: 64 gate + the 64 matching up columns) per CTA, K in steps of
// 64 through a cp.async double buffer, 4 warps x (TM / 4 rows x 64 columns) of mma.sync m16n8k16, fp32
// accumulation; the gated epilogue applies act(gate) * up on the fp32 accumulators.
// TM sorted rows per CTA (64 or 128) on 4 warps of TM / 4 rows x 64 columns: long portions take
// the larger tile, where every weight fragment read from shared memory feeds two row fragments.
constexpr int kTN = 64, kTK = 64, kTLd = kTK + 8;

template <typename T, int MODE, int TM>
__global__ void __launch_bounds__(128)
moe_grouped_gemm_mma_kernel(const T* __restrict__ a, int64_t lda, const T* __restrict__ w, int64_t ldw,
                            int64_t w_expert_stride, const int* __restrict__ offsets,
                            const int* __restrict__ sorted_rows, int E, int top, int Nout, int K,
                            T* __restrict__ out, int64_t ldo, int act,
                            const float* __restrict__ row_scale) {
  constexpr bool GATED = MODE == 1;
  constexpr bool GATHER = MODE != 0;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  constexpr int NB = GATED ? 2 * kTN : kTN;
  constexpr int NT = 128;                            // 4 warps
  constexpr int RW = TM / 64;                        // 16-row fragments per warp
  T* As = reinterpret_cast<T*>(smem_raw);            // [2][TM][kTLd]
  T* Bs = As + 2 * TM * kTLd;                       // [2][NB][kTLd]
  __shared__ int rows[TM];
  int e = 0, tile = blockIdx.x, lo = 0, hi = 0;
  for (; e < E; ++e) {
    lo = offsets[e];
    hi = offsets[e + 1];
    const int nt = (hi - lo + TM - 1) / TM;
    if (tile < nt) break;
    tile -= nt;
  }
  if (e >= E) return;
  const int m0 = lo + tile * TM, mcount = min(TM, hi - m0);
  const int n0 = blockIdx.y * kTN;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < TM) rows[tid] = tid < mcount ? sorted_rows[m0 + tid] : -1;
  __syncthreads();
  const T* we = w + e * w_expert_stride;
  auto load_tile = [&](int k0, int buf) {
    T* ad = As + buf * TM * kTLd;
    for (int c = tid; c < TM * (kTK / 8); c += NT) {
      const int r = c >> 3, ch = c & 7;
      T* d = ad + r * kTLd + ch * 8;
      if (r < mcount && k0 + ch * 8 < K) {
        const int64_t src = GATHER ? rows[r] / top : m0 + r;
        cp_async16(smem_u32(d), a + src * lda + k0 + ch * 8);
      } else {
        *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
      }
    }
    T* bd = Bs + buf * NB * kTLd;
    for (int c = tid; c < NB * (kTK / 8); c += NT) {
      const int r = c >> 3, ch = c & 7;
      const int half = r / kTN, n = n0 + (r - half * kTN);
      T* d = bd + r * kTLd + ch * 8;
      if (n < Nout && k0 + ch * 8 < K)
        cp_async16(smem_u32(d), we + (static_cast<int64_t>(half) * Nout + n) * ldw + k0 + ch * 8);
      else
        *reinterpret_cast<uint4*>(d) = make_uint4(0, 0, 0, 0);
    }
    cp_async_commit();
  };
  float acc[RW][8][4], acc2[RW][GATED ? 8 : 1][4];
#pragma unroll
  for (int f = 0; f < RW; ++f) {
#pragma unroll
    for (int n = 0; n < 8; ++n) acc[f][n][0] = acc[f][n][1] = acc[f][n][2] = acc[f][n][3] = 0.f;
#pragma unroll
    for (int n = 0; n < (GATED ? 8 : 1); ++n)
      acc2[f][n][0] = acc2[f][n][1] = acc2[f][n][2] = acc2[f][n][3] = 0.f;
  }
  const int nk = (K + kTK - 1) / kTK;
  load_tile(0, 0);
  for (int kt = 0; kt < nk; ++kt) {
    cp_async_wait<0>();
    __syncthreads();
    if (kt + 1 < nk) load_tile((kt + 1) * kTK, (kt + 1) & 1);
    const T* at = As + (kt & 1) * TM * kTLd;
    const T* bt = Bs + (kt & 1) * NB * kTLd;
    const uint32_t a_base = smem_u32(at + (warp * 16 * RW + (lane & 15)) * kTLd + (lane >> 4) * 8);
    const uint32_t b_base = smem_u32(bt + ((lane & 7) + ((lane >> 4) << 3)) * kTLd + ((lane >> 3) & 1) * 8);
#pragma unroll
    for (int ks = 0; ks < kTK; ks += 16) {
      uint32_t af[RW][4];
#pragma unroll
      for (int f = 0; f < RW; ++f)
        ldsm_x4(af[f][0], af[f][1], af[f][2], af[f][3], a_base + (f * 16 * kTLd + ks) * 2);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, b_base + (np * 16 * kTLd + ks) * 2);
#pragma unroll
        for (int f = 0; f < RW; ++f) {
          mma16816<T>(acc[f][2 * np], af[f], b0, b1);
          mma16816<T>(acc[f][2 * np + 1], af[f], b2, b3);
        }
        if (GATED) {
          ldsm_x4(b0, b1, b2, b3, b_base + ((kTN + np * 16) * kTLd + ks) * 2);
#pragma unroll
          for (int f = 0; f < RW; ++f) {
            mma16816<T>(acc2[f][GATED ? 2 * np : 0], af[f], b0, b1);
            mma16816<T>(acc2[f][GATED ? 2 * np + 1 : 0], af[f], b2, b3);
          }
        }
      }
    }
  }
  const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
  for (int f = 0; f < RW; ++f)
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int lr = warp * 16 * RW + f * 16 + g + 8 * i;
      if (lr >= mcount) continue;
      const int64_t orow = GATHER ? m0 + lr : rows[lr];
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = n0 + n * 8 + 2 * t4 + c;
          if (col >= Nout) continue;
          float v = acc[f][n][2 * i + c];
          if (GATED) v = moe_act(v, act) * acc2[f][GATED ? n : 0][2 * i + c];
          else if (MODE == 2) v = moe_act(row_scale ? v * row_scale[rows[lr]] : v, act);
          out[orow * ldo + col] = from_float<T>(v);
        }
    }
}

}  // namespace b200

extern "C" int b200_moe_route_scored(const void* h, int64_t ldh, const float* wr, const float* br,
                                     int E, int W, int top, const float* wsg, int* ids, float* wts,
                                     float* gate, int T, int score, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(h && wr && ids && wts, "b200_moe_route: null pointer");
  B200_REQUIRE(E > 0 && E <= 32 * kMaxExpertsPerLane && top > 0 && top <= E && top <= 32 && W > 0,
               "b200_moe_route: experts %d (max %d), top %d", E, 32 * kMaxExpertsPerLane, top);
  B200_REQUIRE(score == 0 || score == 1, "b200_moe_route: score mode %d", score);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("moe_route", st);
  const dim3 grid(T);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(moe_route_kernel<TT>, grid, dim3(256), 0, st, 1, 0, static_cast<const TT*>(h), ldh,  \
                wr, br, E, W, top, wsg, ids, wts, gate, T, score)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_moe_route: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("moe_route_kernel");
  return 0;
}

extern "C" int b200_moe_route(const void* h, int64_t ldh, const float* wr, const float* br, int E,
                              int W, int top, const float* wsg, int* ids, float* wts, float* gate,
                              int T, int dtype, void* stream) {
  return b200_moe_route_scored(h, ldh, wr, br, E, W, top, wsg, ids, wts, gate, T, 0, dtype, stream);
}

extern "C" int b200_moe_align(const int* ids, int N, int E, int* offsets, int* sorted_rows,
                              void* stream) {
  using namespace b200;
  B200_REQUIRE(ids && offsets && sorted_rows && N >= 0 && E > 0 && E <= 4096, "b200_moe_align: bad arguments");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("moe_align", st);
  launch_kernel(moe_align_kernel, dim3(1), dim3(1024), static_cast<size_t>(E + 1) * 4, st, 1, 0, ids,
                N, E, offsets, sorted_rows);
  B200_CHECK_LAUNCH("moe_align_kernel");
  return 0;
}

// mode 0: plain, 1: gated, 2: one weight + activation of the (optionally row-scaled) accumulator
extern "C" int b200_moe_grouped_gemm_mode(const void* a, int64_t lda, const void* w, int64_t ldw,
                                          int64_t w_expert_stride, const int* offsets,
                                          const int* sorted_rows, int E, int top, int rows, int Nout,
                                          int K, void* out, int64_t ldo, int mode, int act,
                                          const float* row_scale, int dtype, void* stream) {
  using namespace b200;
  if (rows == 0) return 0;
  B200_REQUIRE(a && w && offsets && sorted_rows && out, "b200_moe_grouped_gemm: null pointer");
  B200_REQUIRE(E > 0 && top > 0 && rows > 0 && Nout > 0 && K > 0 && act >= 0 && act <= 2 && mode >= 0 &&
                   mode <= 2,
               "b200_moe_grouped_gemm: bad sizes");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("moe_grouped_gemm", st);
  if ((dtype == B200_BF16 || dtype == B200_F16) && K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0 &&
      w_expert_stride % 8 == 0 && aligned16(a) && aligned16(w)) {
    // 128-row tiles once the experts average two of them; every expert can leave one partly filled tile
    const int tm = rows >= 256 * E ? 128 : 64;
    const dim3 tgrid(ceil_div(rows, tm) + min(E, rows), ceil_div(Nout, kTN));
    const size_t smem = static_cast<size_t>(2 * tm + 2 * (mode == 1 ? 2 : 1) * kTN) * kTLd * 2;
#define LAUNCH_TM(TT, G, TMV)                                                                        \
  do {                                                                                               \
    auto kern = moe_grouped_gemm_mma_kernel<TT, G, TMV>;                                             \
    if (smem > 48 * 1024)                                                                            \
      B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                        static_cast<int>(smem)));                                    \
    launch_kernel(kern, tgrid, dim3(128), smem, st, 1, 0, static_cast<const TT*>(a), lda,            \
                  static_cast<const TT*>(w), ldw, w_expert_stride, offsets, sorted_rows, E, top,     \
                  Nout, K, static_cast<TT*>(out), ldo, act, row_scale);                              \
  } while (0)
#define LAUNCH_TC(TT, G)                                                                             \
  do {                                                                                               \
    if (tm == 128) LAUNCH_TM(TT, G, 128);                                                            \
    else LAUNCH_TM(TT, G, 64);                                                                       \
  } while (0)
#define BY_MODE(TT)                    \
  do {                                 \
    if (mode == 1) LAUNCH_TC(TT, 1);   \
    else if (mode == 2) LAUNCH_TC(TT, 2); \
    else LAUNCH_TC(TT, 0);             \
  } while (0)
    if (dtype == B200_BF16) BY_MODE(__nv_bfloat16);
    else BY_MODE(__half);
#undef BY_MODE
#undef LAUNCH_TC
#undef LAUNCH_TM
    B200_CHECK_LAUNCH("moe_grouped_gemm_mma_kernel");
    note_variant("moe_grouped_gemm_mma gated%d", mode);
    return 0;
  }
  // every expert can leave one partly filled row tile
  const dim3 grid(ceil_div(rows, kGM) + min(E, rows), ceil_div(Nout, kGN));
#define LAUNCH(TT, G)                                                                                \
  launch_kernel(moe_grouped_gemm_kernel<TT, G>, grid, dim3(256), 0, st, 1, 0,                        \
                static_cast<const TT*>(a), lda, static_cast<const TT*>(w), ldw, w_expert_stride,     \
                offsets, sorted_rows, E, top, Nout, K, static_cast<TT*>(out), ldo, act, row_scale)
#define BY_G(TT)                     \
  do {                               \
    if (mode == 1) LAUNCH(TT, 1);    \
    else if (mode == 2) LAUNCH(TT, 2); \
    else LAUNCH(TT, 0);              \
  } while (0)
  if (dtype == B200_BF16) BY_G(__nv_bfloat16);
  else if (dtype == B200_F16) BY_G(__half);
  else if (dtype == B200_F32) BY_G(float);
  else B200_REQUIRE(false, "b200_moe_grouped_gemm: dtype %d", dtype);
#undef BY_G
#undef LAUNCH
  B200_CHECK_LAUNCH("moe_grouped_gemm_kernel");
  return 0;
}

extern "C" int b200_moe_grouped_gemm(const void* a, int64_t lda, const void* w, int64_t ldw,
                                     int64_t w_expert_stride, const int* offsets,
                                     const int* sorted_rows, int E, int top, int rows, int Nout, int K,
                                     void* out, int64_t ldo, int gated, int act, int dtype,
                                     void* stream) {
  return b200_moe_grouped_gemm_mode(a, lda, w, ldw, w_expert_stride, offsets, sorted_rows, E, top, rows,
                                    Nout, K, out, ldo, gated ? 1 : 0, act, nullptr, dtype, stream);
}

extern "C" int b200_moe_route_grouped(const void* h, int64_t ldh, const float* wr, const float* correction,
                                      int E, int W, int top, int n_groups, int keep, int* ids, float* wts,
                                      int T, int dtype, void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(h && wr && ids && wts, "b200_moe_route_grouped: null pointer");
  B200_REQUIRE(E > 0 && E <= 32 * kMaxExpertsPerLane && top > 0 && top <= E && top <= 32 && W > 0,
               "b200_moe_route_grouped: experts %d (max %d), top %d", E, 32 * kMaxExpertsPerLane, top);
  B200_REQUIRE(n_groups >= 1 && E % n_groups == 0 && keep >= 1 && keep <= n_groups &&
                   keep * (E / n_groups) >= top,
               "b200_moe_route_grouped: %d experts in %d groups, %d kept, top %d", E, n_groups, keep, top);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("moe_route", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(moe_route_grouped_kernel<TT>, dim3(T), dim3(256), 0, st, 1, 0,                      \
                static_cast<const TT*>(h), ldh, wr, correction, E, W, top, n_groups, keep, ids, wts)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_moe_route_grouped: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("moe_route_grouped_kernel");
  return 0;
}
