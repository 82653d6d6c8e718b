// Matrix-state linear recurrences over a mixed batch, state in fp32 and carried per sequence:
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T        S [D, E] per head        o_t = S_t^T q_t
//
//   decay form : a_t = decay[head] (constant), b_t = 1                     (decayed linear attention)
//   gated form : log-space input and forget gates with a running stabiliser m (m_0 = 0):
//             li = cap tanh(zi / cap), lf = logsigmoid(cap tanh(zf / cap))   (cap <= 0: no capping)
//             m_t = max(lf + m_(t-1), li), a_t = exp(lf + m_(t-1) - m_t), b_t = exp(li - m_t)
//             and the normaliser n_t = a_t n_(t-1) + b_t k_t, which is the same recurrence for one more
//             value column that is always 1.  The kernel returns the un-normalised o_t together with
//             n_t . q_t and m_t per (token, head); the consumer divides by
//             max(|n_t . q_t|, exp(-m_t)) + den_eps                                          (mLSTM)
//
// One CTA owns (batch entry, head, a slice of the value columns) and walks the entry's new tokens in
// order, so a token's result is the same sum in the same order however the sequence was cut into
// steps.  A thread keeps 16 rows d of TWO neighbouring columns in registers, two ROWS to a 64-bit
// register, so that the pairs (k_d, k_d+1) and (q_d, q_d+1) come straight out of one 16-byte
// shared-memory load and every state element costs 1.5 packed fp32 instructions per token; the P
// lanes that share a column pair add their partial dot products by shuffles.
// The host sizes the CTA: a whole head (up to 512 threads, so q and k are staged once per head and
// every scheduler holds four warps) unless that leaves SMs idle, then the columns are split further.
// Tokens are staged a chunk (up to 32) at a time: the raw q, k, v rows of the NEXT chunk stream into
// shared memory with cp.async while the current chunk is computed, then one pass converts them to
// fp32 (activation, query scale, zero padding to P * 16 rows); rows that are not 8-byte aligned are
// staged with plain loads instead.  The gated form's scalar chain m_t runs once per chunk in one
// lane, the exponentials beside it in parallel.  The state row of a sequence is read when its portion
// does not start at position 0 (there it is zero) and written back at the end; a single decoded token
// is the same kernel with a portion of one.  The state's layout is the kernel's own and does not
// depend on the CTA size: per head, atoms of 4 rows x 2 columns (32 bytes, one sector) ordered
// [column pair][row / 4], then one copy of m per column pair;
// b200_linear_recurrence_state_width gives its size.
//
//   gated_group_rmsnorm : out = o / sqrt(mean_group(o^2) + eps) * w * sigmoid(z), the mean taken over
//                         consecutive groups of `group` coordinates (one head, or the whole row);
//                         with the gated form's (n . q, m) per head, o is first divided as above.
//                         Gate mode 1: o is multiplied by silu(z) BEFORE the norm instead.
#include <cstdlib>

#include "common.cuh"

namespace b200 {

constexpr int kRecMaxThreads = 512;
constexpr int kRecMaxRows = 16;  // rows of S per thread: 8 (key size <= 256) or 16; D <= rows * P, P <= 32
constexpr int kRecChunk = 32;    // most tokens staged in shared memory at a time

__device__ __forceinline__ float rec_act(float z, int act) {
  return act == 1 ? z / (1.0f + expf(-z)) : z;
}
__device__ __forceinline__ void cp_async8(uint32_t smem_addr, const void* gptr) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(smem_addr), "l"(gptr));
}
// two fp32 lanes in one 64-bit register: the packed multiply-adds below take and return these, so no
// instruction is spent on pairing registers
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};\n" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;\n" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;\n" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;\n" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float log_sigmoid(float z) {
  return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

template <typename T, bool GATES, int kRecRows>
__global__ void __launch_bounds__(kRecMaxThreads)
linear_recurrence_kernel(const T* __restrict__ q, int64_t ldq, const T* __restrict__ k, int64_t ldk,
                         const T* __restrict__ v, int64_t ldv, const float* __restrict__ gates,
                         int64_t ldg, const float* __restrict__ decay, float cap, float q_scale,
                         int act, float* __restrict__ state, int64_t ld_state,
                         const int64_t* __restrict__ slot, const int* __restrict__ tok_pos,
                         const int* __restrict__ ext_start, const int* __restrict__ ext_len,
                         float* __restrict__ out, int64_t ldo, float* __restrict__ aux, int64_t ld_aux,
                         int H, int D, int E, int P, int CH, int stream_rows) {
  extern __shared__ __align__(16) float rec_smem[];
  const int nthreads = blockDim.x, nwarps = nthreads >> 5;
  const int Dp = P * kRecRows;                // padded key size
  const int ES = 2 * (nthreads / P);          // value columns of this CTA
  float* qs = rec_smem;                       // [CH][Dp]
  float* ks = qs + CH * Dp;                   // [CH][Dp]
  float* vs = ks + CH * Dp;                   // [CH][ES]
  float* ga = vs + CH * ES;                   // [32] a_t
  float* gb = ga + kRecChunk;                 // [32] b_t
  float* gm = gb + kRecChunk;                 // [32] m_t
  float* gl = gm + kRecChunk;                 // [2][32] li, lf
  // raw rows in flight, two stages of [CH][2 D + ES] values of T (8-byte pieces)
  T* raw = reinterpret_cast<T*>(gl + 2 * kRecChunk);
  const int raw_stage = CH * (2 * D + ES);
  const int b = blockIdx.z, h = blockIdx.y, e0 = blockIdx.x * ES;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int p = tid % P, cp = tid / P, e = e0 + 2 * cp;
  const int start = ext_start[b], len = ext_len[b];
  if (len <= 0) return;
  const bool fresh = tok_pos[start] == 0;
  const int ncols = E + (GATES ? 1 : 0);      // the gated form's last column is the normaliser (v = 1)
  const int NCP = (ncols + 1) / 2, D4 = (D + 3) / 4;
  const int64_t head_width = static_cast<int64_t>(D4) * NCP * 8 + (GATES ? (NCP + 7) / 8 * 8 : 0);
  float* st = state + slot[b] * ld_state + h * head_width;
  float* st_m = st + static_cast<int64_t>(D4) * NCP * 8;
  const int cpg = blockIdx.x * (nthreads / P) + cp;      // column pair within the head
  // this thread's rows: atoms (4 rows) number a * P + p, a < 4, so that the lanes of a column pair
  // touch consecutive atoms in the state and consecutive float4 of the staged q and k
  // s0 / s1: first / second column; entry 2 a + i holds rows (4 d4 + 2 i, 4 d4 + 2 i + 1) of atom a.
  // An atom in memory is [row][column]: (r0c0, r0c1, r1c0, r1c1), (r2c0, r2c1, r3c0, r3c1).
  f32x2 s0[kRecRows / 2], s1[kRecRows / 2];
#pragma unroll
  for (int a4 = 0; a4 < kRecRows / 4; ++a4) {
    const int d4 = a4 * P + p;
    float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
    if (!fresh && d4 < D4 && cpg < NCP) {
      const float4* at = reinterpret_cast<const float4*>(st + (static_cast<int64_t>(cpg) * D4 + d4) * 8);
      v0 = at[0];
      v1 = at[1];
    }
    s0[2 * a4] = pack2(v0.x, v0.z);
    s1[2 * a4] = pack2(v0.y, v0.w);
    s0[2 * a4 + 1] = pack2(v1.x, v1.z);
    s1[2 * a4 + 1] = pack2(v1.y, v1.w);
  }
  float m = (GATES && !fresh) ? st_m[min(cpg, NCP - 1)] : 0.f;
  const float lam = GATES ? 0.f : decay[h];
  const int vvalid = max(0, min(ES, E - e0));  // value columns of this slice that exist
  constexpr int PE = 8 / sizeof(T);            // values per 8-byte piece
  auto issue_chunk = [&](int c0, int stage) {
    const int n = min(CH, len - c0);
    T* rq = raw + stage * raw_stage;
    T* rk = rq + CH * D;
    T* rv = rk + CH * D;
    const int dp = D / PE, vp = vvalid / PE;
    for (int j = warp; j < n; j += nwarps) {
      const int64_t row = start + c0 + j;
      for (int c = lane; c < dp; c += 32) {
        cp_async8(smem_u32(rq + j * D + c * PE), q + row * ldq + h * D + c * PE);
        cp_async8(smem_u32(rk + j * D + c * PE), k + row * ldk + h * D + c * PE);
      }
      for (int c = lane; c < vp; c += 32)
        cp_async8(smem_u32(rv + j * ES + c * PE), v + row * ldv + h * E + e0 + c * PE);
    }
    cp_async_commit();
  };
  float gi_next = 0.f, gf_next = 0.f;          // gate pre-activations of the next chunk (warp 0)
  auto load_gates = [&](int c0) {
    if (GATES && tid < 32 && c0 + tid < len) {
      const int64_t row = start + c0 + tid;
      gi_next = gates[row * ldg + h];
      gf_next = gates[row * ldg + H + h];
    }
  };
  if (stream_rows) issue_chunk(0, 0);
  load_gates(0);
  for (int c0 = 0; c0 < len; c0 += CH) {
    const int n = min(CH, len - c0);
    const int stage = (c0 / CH) & 1;
    if (stream_rows) {
      if (c0 + CH < len) {
        issue_chunk(c0 + CH, stage ^ 1);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
    }
    __syncthreads();
    const T* rq = raw + stage * raw_stage;
    const T* rk = rq + CH * D;
    const T* rv = rk + CH * D;
    for (int j = warp; j < n; j += nwarps) {
      const int64_t row = start + c0 + j;
      for (int d = lane; d < Dp; d += 32) {
        float qv = 0.f, kv = 0.f;
        if (d < D) {
          qv = to_float<T>(stream_rows ? rq[j * D + d] : q[row * ldq + h * D + d]);
          kv = to_float<T>(stream_rows ? rk[j * D + d] : k[row * ldk + h * D + d]);
          qv = rec_act(qv, act) * q_scale;
          kv = rec_act(kv, act);
        }
        qs[j * Dp + d] = qv;
        ks[j * Dp + d] = kv;
      }
      for (int c = lane; c < ES; c += 32) {
        float x = 0.f;
        if (e0 + c < E)
          x = rec_act(to_float<T>(stream_rows ? rv[j * ES + c] : v[row * ldv + h * E + e0 + c]), act);
        else if (GATES && e0 + c == E) x = 1.f;
        vs[j * ES + c] = x;
      }
    }
    if (GATES && tid < 32) {
      // gate values of the chunk in parallel, the stabiliser chain in one lane, the exponentials
      // in parallel again
      float li = 0.f, lf = 0.f;
      if (tid < n) {
        li = gi_next;
        lf = gf_next;
        if (cap > 0.f) {
          li = cap * tanhf(li / cap);
          lf = cap * tanhf(lf / cap);
        }
        lf = log_sigmoid(lf);
        gl[tid] = li;
        gl[kRecChunk + tid] = lf;
      }
      __syncwarp();
      if (tid == 0) {
        float mm = m;
        for (int j = 0; j < n; ++j) {
          mm = fmaxf(gl[kRecChunk + j] + mm, gl[j]);
          gm[j] = mm;
        }
      }
      __syncwarp();
      if (tid < n) {
        const float mp = tid == 0 ? m : gm[tid - 1];
        ga[tid] = expf(lf + mp - gm[tid]);
        gb[tid] = expf(li - gm[tid]);
      }
    }
    __syncthreads();
    load_gates(c0 + CH);                      // in flight during this chunk's tokens
    if (GATES) {
      m = gm[n - 1];
      if (aux && blockIdx.x == 0 && tid < n) aux[(start + c0 + tid) * ld_aux + H + h] = gm[tid];
    }
#pragma unroll 2
    for (int j = 0; j < n; ++j) {
      const float a = GATES ? ga[j] : lam, bb = GATES ? gb[j] : 1.f;
      const f32x2 a2 = pack2(a, a);
      const float2 vv = *reinterpret_cast<const float2*>(vs + j * ES + 2 * cp);
      const f32x2 ve0 = pack2(vv.x * bb, vv.x * bb), ve1 = pack2(vv.y * bb, vv.y * bb);
      const ulonglong2* k4 = reinterpret_cast<const ulonglong2*>(ks + j * Dp) + p;
      const ulonglong2* q4 = reinterpret_cast<const ulonglong2*>(qs + j * Dp) + p;
      f32x2 acc0a = 0ull, acc0b = 0ull, acc1a = 0ull, acc1b = 0ull;   // 0.0f twice
#pragma unroll
      for (int r4 = 0; r4 < kRecRows / 4; ++r4) {
        const ulonglong2 kk = k4[r4 * P], qq = q4[r4 * P];     // rows 4 d4 .. 4 d4 + 3 as two row pairs
        s0[2 * r4] = fma2(a2, s0[2 * r4], mul2(kk.x, ve0));
        acc0a = fma2(s0[2 * r4], qq.x, acc0a);
        s1[2 * r4] = fma2(a2, s1[2 * r4], mul2(kk.x, ve1));
        acc1a = fma2(s1[2 * r4], qq.x, acc1a);
        s0[2 * r4 + 1] = fma2(a2, s0[2 * r4 + 1], mul2(kk.y, ve0));
        acc0b = fma2(s0[2 * r4 + 1], qq.y, acc0b);
        s1[2 * r4 + 1] = fma2(a2, s1[2 * r4 + 1], mul2(kk.y, ve1));
        acc1b = fma2(s1[2 * r4 + 1], qq.y, acc1b);
      }
      float x0, x1, x2, x3, y0, y1, y2, y3;
      unpack2(acc0a, x0, x1);
      unpack2(acc0b, x2, x3);
      unpack2(acc1a, y0, y1);
      unpack2(acc1b, y2, y3);
      float ax = (x0 + x1) + (x2 + x3), ay = (y0 + y1) + (y2 + y3);
      for (int o = P >> 1; o > 0; o >>= 1) {
        ax += __shfl_xor_sync(0xffffffffu, ax, o);
        ay += __shfl_xor_sync(0xffffffffu, ay, o);
      }
      if (p == 0) {
        const int64_t row = start + c0 + j;
        if (e < E) out[row * ldo + h * E + e] = ax;
        else if (GATES && e == E && aux) aux[row * ld_aux + h] = ax;
        if (e + 1 < E) out[row * ldo + h * E + e + 1] = ay;
        else if (GATES && e + 1 == E && aux) aux[row * ld_aux + h] = ay;
      }
    }
  }
#pragma unroll
  for (int a4 = 0; a4 < kRecRows / 4; ++a4) {
    const int d4 = a4 * P + p;
    if (d4 < D4 && cpg < NCP) {
      float4* at = reinterpret_cast<float4*>(st + (static_cast<int64_t>(cpg) * D4 + d4) * 8);
      float4 v0, v1;
      unpack2(s0[2 * a4], v0.x, v0.z);
      unpack2(s1[2 * a4], v0.y, v0.w);
      unpack2(s0[2 * a4 + 1], v1.x, v1.z);
      unpack2(s1[2 * a4 + 1], v1.y, v1.w);
      at[0] = v0;
      at[1] = v1;
    }
  }
  if (GATES && p == 0 && cpg < NCP) st_m[cpg] = m;
}

template <typename TZ, typename TO>
__global__ void __launch_bounds__(256)
gated_group_rmsnorm_kernel(const float* __restrict__ o, int64_t ldo, const float* __restrict__ w,
                           const TZ* __restrict__ z, int64_t ldz, TO* __restrict__ out, int64_t ldout,
                           int N, int group, float eps, const float* __restrict__ aux, int64_t ld_aux,
                           int H, float den_eps, int gate_mode) {
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* row = o + t * ldo;
  const int head_size = aux ? N / H : 1;
  for (int g0 = warp * group; g0 < N; g0 += 8 * group) {
    float ss = 0.f;
    for (int d = lane; d < group; d += 32) {
      float x = row[g0 + d];
      if (aux) {
        const int hd = (g0 + d) / head_size;
        x /= fmaxf(fabsf(aux[t * ld_aux + hd]), expf(-aux[t * ld_aux + H + hd])) + den_eps;
      }
      if (gate_mode == 1) {                     // the gate silu(z) multiplies BEFORE the norm
        const float zz = to_float<TZ>(z[t * ldz + g0 + d]);
        x *= zz / (1.0f + expf(-zz));
      }
      ss = fmaf(x, x, ss);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float r = 1.0f / sqrtf(ss / static_cast<float>(group) + eps);
    for (int d = lane; d < group; d += 32) {
      float y = row[g0 + d] * r;
      if (aux) {
        const int hd = (g0 + d) / head_size;
        y /= fmaxf(fabsf(aux[t * ld_aux + hd]), expf(-aux[t * ld_aux + H + hd])) + den_eps;
      }
      if (w) y *= w[g0 + d];
      if (z) {
        const float zz = to_float<TZ>(z[t * ldz + g0 + d]);
        y *= gate_mode == 1 ? zz / (1.0f + expf(-zz)) : 1.0f / (1.0f + expf(-zz));
      }
      out[t * ldout + g0 + d] = from_float<TO>(y);
    }
  }
}

}  // namespace b200

static int rec_parts(int D, int rows) {
  int P = 1;
  while (rows * P < D) P <<= 1;
  return P;
}
static int64_t rec_head_width(int D, int E, int gated) {
  const int64_t ncp = (E + (gated ? 1 : 0) + 1) / 2, d4 = (D + 3) / 4;
  return d4 * ncp * 8 + (gated ? (ncp + 7) / 8 * 8 : 0);
}

// fp32 values one sequence keeps per layer (the layout is the kernel's own)
extern "C" int64_t b200_linear_recurrence_state_width(int H, int D, int E, int gated) {
  if (H <= 0 || D <= 0 || E <= 0 || D > b200::kRecMaxRows * 32) return -1;
  return static_cast<int64_t>(H) * rec_head_width(D, E, gated);
}

extern "C" int b200_linear_recurrence(const void* q, int64_t ldq, const void* k, int64_t ldk,
                                      const void* v, int64_t ldv, const float* gates, int64_t ldg,
                                      const float* decay, float cap, float q_scale, int act,
                                      float* state, int64_t ld_state, const int64_t* slot,
                                      const int* tok_pos, const int* ext_start, const int* ext_len,
                                      float* out, int64_t ldo, float* aux, int64_t ld_aux, int batch,
                                      int H, int D, int E, int dtype, void* stream) {
  using namespace b200;
  if (batch == 0) return 0;
  B200_REQUIRE(q && k && v && state && slot && tok_pos && ext_start && ext_len && out,
               "b200_linear_recurrence: null pointer");
  B200_REQUIRE((gates != nullptr) != (decay != nullptr),
               "b200_linear_recurrence: give either gate pre-activations or a decay per head");
  B200_REQUIRE(!gates || aux, "b200_linear_recurrence: the gated form returns (n . q, m) in aux");
  B200_REQUIRE(batch > 0 && H > 0 && D > 0 && E > 0 && D <= kRecMaxRows * 32 && (act == 0 || act == 1),
               "b200_linear_recurrence: heads %d, key size %d (max %d), value size %d", H, D,
               kRecMaxRows * 32, E);
  B200_REQUIRE(ld_state % 4 == 0 && aligned16(state),
               "b200_linear_recurrence: the state rows must be 16-byte aligned");
  B200_REQUIRE(H <= 65535 && batch <= 65535, "b200_linear_recurrence: grid too large");
  const int ncols = E + (gates ? 1 : 0), ncp = (ncols + 1) / 2;
  // 16 rows per thread; the 8-row instance (twice the warps per head) measured slower at every size
  const int kRecRows = 16;
  const int P = rec_parts(D, kRecRows);
  // column pairs per CTA: a whole head if 512 threads hold it; split further while the grid is
  // smaller than the GPU
  int pairs = kRecMaxThreads / P;
  while (pairs / 2 >= ncp && pairs * P > 32) pairs /= 2;        // no idle half
  // (measured: below four warps per CTA a split no longer pays; B200_REC_MIN_THREADS overrides for A/B runs)
  static const int min_threads = [] {
    const char* e = std::getenv("B200_REC_MIN_THREADS");
    return (e && *e) ? std::atoi(e) : 128;
  }();
  while (static_cast<int64_t>(batch) * H * ceil_div(ncp, pairs) < device_sm_count() && pairs * P > min_threads)
    pairs /= 2;
  const int nthreads = pairs * P, ES = 2 * pairs;
  const size_t esz = dtype == B200_F32 ? 4 : 2;
  // rows stream through cp.async in 8-byte pieces when every piece is aligned
  const int pe = static_cast<int>(8 / esz);
  const bool stream_rows = D % pe == 0 && E % pe == 0 && ldq % pe == 0 && ldk % pe == 0 && ldv % pe == 0 &&
                           ES % pe == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0 &&
                           (reinterpret_cast<uintptr_t>(k) & 7) == 0 && (reinterpret_cast<uintptr_t>(v) & 7) == 0;
  auto smem_for = [&](int ch) {
    return sizeof(float) * (static_cast<size_t>(ch) * (2 * P * kRecRows + ES) + 5 * kRecChunk) +
           (stream_rows ? 2 * esz * ch * (2 * D + ES) : 0);
  };
  int CH = kRecChunk;
  while (CH > 4 && smem_for(CH) > 100 * 1024) CH >>= 1;   // two CTAs per SM
  const size_t smem = smem_for(CH);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("linear_recurrence", st);
  const dim3 grid(ceil_div(ncp, pairs), H, batch);
#define LAUNCH(TT, G)               \
  do {                              \
    if (kRecRows == 8) LAUNCH_R(TT, G, 8); \
    else LAUNCH_R(TT, G, 16);       \
  } while (0)
#define LAUNCH_R(TT, G, RR)                                                                          \
  do {                                                                                               \
    auto kern = linear_recurrence_kernel<TT, G, RR>;                                                 \
    if (smem > 48 * 1024)                                                                            \
      B200_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,           \
                                        static_cast<int>(smem)));                                    \
    launch_kernel(kern, grid, dim3(nthreads), smem, st, 1, 0, static_cast<const TT*>(q), ldq,        \
                  static_cast<const TT*>(k), ldk, static_cast<const TT*>(v), ldv, gates, ldg, decay, \
                  cap, q_scale, act, state, ld_state, slot, tok_pos, ext_start, ext_len, out, ldo,   \
                  aux, ld_aux, H, D, E, P, CH, stream_rows ? 1 : 0);                                 \
  } while (0)
#define BY_G(TT)                  \
  do {                            \
    if (gates) LAUNCH(TT, true);  \
    else LAUNCH(TT, false);       \
  } while (0)
  if (dtype == B200_BF16) BY_G(__nv_bfloat16);
  else if (dtype == B200_F16) BY_G(__half);
  else if (dtype == B200_F32) BY_G(float);
  else B200_REQUIRE(false, "b200_linear_recurrence: dtype %d", dtype);
#undef BY_G
#undef LAUNCH
#undef LAUNCH_R
  note_variant("linear_recurrence rows%d threads%d parts%d chunk%d stream%d", kRecRows, nthreads, P, CH, stream_rows ? 1 : 0);
  B200_CHECK_LAUNCH("linear_recurrence_kernel");
  return 0;
}

// aux (optional): fp32 [T, 2 H] = (n . q, m) of the gated recurrence; o is divided by
// max(|n . q|, exp(-m)) + den_eps per (token, head) before the norm
extern "C" int b200_gated_group_rmsnorm_mode(const float* o, int64_t ldo, const float* w, const void* z,
                                             int64_t ldz, void* out, int64_t ldout, int T, int N,
                                             int group, float eps, const float* aux, int64_t ld_aux,
                                             int H, float den_eps, int gate_mode, int dtype,
                                             void* stream) {
  using namespace b200;
  if (T == 0) return 0;
  B200_REQUIRE(gate_mode == 0 || (gate_mode == 1 && z), "b200_gated_group_rmsnorm: gate mode %d", gate_mode);
  B200_REQUIRE(o && out && T > 0 && N > 0 && group > 0 && N % group == 0,
               "b200_gated_group_rmsnorm: %d coordinates in groups of %d", N, group);
  B200_REQUIRE(!aux || (H > 0 && N % H == 0), "b200_gated_group_rmsnorm: %d coordinates, %d heads", N, H);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ScopedKernelTimer timer("gated_group_rmsnorm", st);
#define LAUNCH(TT)                                                                                   \
  launch_kernel(gated_group_rmsnorm_kernel<TT, TT>, dim3(T), dim3(256), 0, st, 1, 0, o, ldo, w,      \
                static_cast<const TT*>(z), ldz, static_cast<TT*>(out), ldout, N, group, eps, aux,    \
                ld_aux, H, den_eps, gate_mode)
  if (dtype == B200_BF16) LAUNCH(__nv_bfloat16);
  else if (dtype == B200_F16) LAUNCH(__half);
  else if (dtype == B200_F32) LAUNCH(float);
  else B200_REQUIRE(false, "b200_gated_group_rmsnorm: dtype %d", dtype);
#undef LAUNCH
  B200_CHECK_LAUNCH("gated_group_rmsnorm_kernel");
  return 0;
}

extern "C" int b200_gated_group_rmsnorm(const float* o, int64_t ldo, const float* w, const void* z,
                                        int64_t ldz, void* out, int64_t ldout, int T, int N,
                                        int group, float eps, const float* aux, int64_t ld_aux, int H,
                                        float den_eps, int dtype, void* stream) {
  return b200_gated_group_rmsnorm_mode(o, ldo, w, z, ldz, out, ldout, T, N, group, eps, aux, ld_aux, H,
                                       den_eps, 0, dtype, stream);
}
