// The matrix-state recurrences of recurrent.cu for prompt portions, in chunks of 64 tokens.
//
// Walking a portion token by token is a chain of T dependent steps per head.  Here the chain has one
// link per chunk.  With L_i the running sum, inside the chunk, of the logarithms of the decays up to
// and including token i (one per key channel; for the decayed sum L_i = (i + 1) log a), k and q as
// the recurrence uses them (unit length, or silu), S_0 the state before the chunk:
//
//   every write u_j reaches token i >= j weakened by exp(L_i - L_j) <= 1:
//     S_i = diag(exp L_i) S_0 + sum_{j<=i} diag(exp(L_i - L_j)) k_j u_j^T
//   decayed sum: u_j = v_j.   Delta rule: u_j = beta_j (v_j - k_j^T diag(g_j) S_{j-1}), which, with
//     A_jm = sum_c k_j[c] k_m[c] exp(L_j[c] - L_m[c])  (m < j),    T = I + diag(beta) A,
//     is the triangular system  T U = diag(beta) (V - (K * exp L) S_0),  so
//     U = Uv - W S_0  with  Uv = T^-1 diag(beta) V  and  W = T^-1 diag(beta) (K * exp L),
//     two matrices that do not depend on the state.
//   read-out: o_i = (q_i * exp L_i)^T S_0 + sum_{j<=i} B_ij u_j,   B_ij = sum_c q_i[c] k_j[c] exp(L_i[c] - L_j[c])
//   state after the chunk of n tokens: S = diag(exp L_{n-1}) S_0 + (K * exp(L_{n-1} - L))^T U
//
// Only differences L_i - L_j with i >= j are ever exponentiated, so nothing overflows however strong
// the decay.  Two launches: `chunk_prepare` makes W, Uv, B, Q * exp L, K * exp(L_end - L) and exp L_end
// for every (chunk, head) in parallel; `chunk_apply` walks each sequence's chunks in order, a block per
// (sequence, head, 16 state columns), with three small matrix products per chunk.  All arithmetic is
// float on the CUDA cores: scores, decays, the triangular solve and the state stay 32-bit in both
// storage types.  Chunks start at the portion's first token; results do not depend on where a
// portion is cut beyond rounding.
#include "common.cuh"

namespace pmm {

constexpr int kChunk = 64;
constexpr int kPrepThreads = 256;
constexpr int kApplyThreads = 128;
constexpr int kApplyCols = 16;

__device__ __forceinline__ float sigmoid_c(float x) { return 1.f / (1.f + expf(-x)); }

struct ChunkArgs {
  const void* q; long long ld_q;        // [T, Hk*d]
  const void* k; long long ld_k;
  const void* v; long long ld_v;        // [T, H*dv]
  const void* beta; long long ld_beta;  // delta: [T, H]
  const void* a; long long ld_a;        // delta: [T, H*d]
  const float* dt_bias; const float* a_log; const float* decay;
  const int* cu; int n_seq;
  int H, Hk, d, dv;
  float unit_eps, q_scale;
  // per (chunk, head), chunk-major: W [C, d] (delta), Uv [C, dv], B [C, C], Qg [C, d], Ke [C, d], Eg [d]
  float *W, *Uv, *B, *Qg, *Ke, *Eg;
  float* state; const int* slots; float* out;
};

// chunk index -> (sequence, first token, tokens in the chunk); false for a surplus block
__device__ __forceinline__ bool locate_chunk(const int* __restrict__ cu, int n_seq, int chunk, int* seq, int* t0, int* n) {
  int base = 0;
  for (int s = 0; s < n_seq; ++s) {
    const int len = cu[s + 1] - cu[s];
    const int nc = (len + kChunk - 1) / kChunk;
    if (chunk < base + nc) {
      const int local = chunk - base;
      *seq = s;
      *t0 = cu[s] + local * kChunk;
      *n = min(kChunk, len - local * kChunk);
      return true;
    }
    base += nc;
  }
  return false;
}

template <typename S, bool DELTA>
__global__ void __launch_bounds__(kPrepThreads)
    chunk_prepare_kernel(ChunkArgs p) {
  extern __shared__ float sm[];
  const int d = p.d, dv = p.dv, ds = d + 1;  // rows of stride d + 1: row i, column c sits in bank (i + c) mod 32
  float* sK = sm;                         // [C][ds]
  float* sQ = sK + kChunk * ds;           // [C][ds]   (later: the right-hand sides of the solve)
  float* sL = sQ + kChunk * ds;           // delta: [C][ds]
  float* sA = sL + (DELTA ? kChunk * ds : 0);  // delta: [C][C + 1]
  __shared__ float s_beta[kChunk];
  pdl_launch_dependents();
  pdl_wait();
  const int chunk = blockIdx.x, h = blockIdx.y;
  int seq, t0, n;
  if (!locate_chunk(p.cu, p.n_seq, chunk, &seq, &t0, &n)) return;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const S* gq = static_cast<const S*>(p.q);
  const S* gk = static_cast<const S*>(p.k);
  const S* gv = static_cast<const S*>(p.v);
  const size_t ch = static_cast<size_t>(chunk) * p.H + h;
  float* oW = p.W + ch * kChunk * d;
  float* oUv = p.Uv + ch * kChunk * dv;
  float* oB = p.B + ch * kChunk * kChunk;
  float* oQg = p.Qg + ch * kChunk * d;
  float* oKe = p.Ke + ch * kChunk * d;
  float* oEg = p.Eg + ch * d;

  // ---- q, k (and the logarithms of the decays) of the chunk's tokens
  const float a_neg = DELTA ? -expf(p.a_log[h]) : 0.f;
  for (int e = tid; e < n * d; e += kPrepThreads) {
    const int i = e / d, c = e - i * d;
    const long long t = t0 + i;
    const float qv = ldf(gq + t * p.ld_q + hk * d + c), kv = ldf(gk + t * p.ld_k + hk * d + c);
    if (DELTA) {
      sQ[i * ds + c] = qv;
      sK[i * ds + c] = kv;
      const float av = ldf(static_cast<const S*>(p.a) + t * p.ld_a + h * d + c) + p.dt_bias[h * d + c];
      sL[i * ds + c] = a_neg * softplus_f(av);
    } else {
      sQ[i * ds + c] = silu_f(qv);
      sK[i * ds + c] = silu_f(kv);
    }
  }
  if (DELTA && tid < n) s_beta[tid] = sigmoid_c(ldf(static_cast<const S*>(p.beta) + static_cast<long long>(t0 + tid) * p.ld_beta + h));
  __syncthreads();
  const float log_a = DELTA ? 0.f : logf(fmaxf(p.decay[h], 1e-38f));
  if (DELTA) {
    for (int i = warp; i < n; i += kPrepThreads / 32) {  // unit length per token
      float sq = 0.f, sk = 0.f;
      for (int c = lane; c < d; c += 32) {
        sq += sQ[i * ds + c] * sQ[i * ds + c];
        sk += sK[i * ds + c] * sK[i * ds + c];
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float fq = p.q_scale / sqrtf(sq + p.unit_eps), fk = 1.f / sqrtf(sk + p.unit_eps);
      for (int c = lane; c < d; c += 32) {
        sQ[i * ds + c] *= fq;
        sK[i * ds + c] *= fk;
      }
    }
    for (int c = tid; c < d; c += kPrepThreads) {  // running sums of the logarithms
      float run = 0.f;
      for (int i = 0; i < n; ++i) {
        run += sL[i * ds + c];
        sL[i * ds + c] = run;
      }
    }
    __syncthreads();
  }

  // ---- A (delta) and B: a warp takes rows i, a lane the columns j = lane and lane + 32
  for (int i = warp; i < n; i += kPrepThreads / 32) {
    const float* qi = sQ + i * ds;
    const float* ki = sK + i * ds;
    const float* li = sL + i * ds;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int j = lane + 32 * half;
      if (j > i) continue;
      const float* kj = sK + j * ds;
      float accA = 0.f, accB = 0.f;
      if (DELTA) {
        const float* lj = sL + j * ds;
        for (int c = 0; c < d; ++c) {
          const float w = expf(li[c] - lj[c]) * kj[c];
          accA += ki[c] * w;
          accB += qi[c] * w;
        }
        sA[i * (kChunk + 1) + j] = accA;
      } else {
        for (int c = 0; c < d; ++c) accB += qi[c] * kj[c];
        accB *= expf(log_a * static_cast<float>(i - j));
      }
      oB[i * kChunk + j] = accB;
    }
  }
  // ---- q * exp L, k * exp(L_end - L), exp L_end
  for (int e = tid; e < n * d; e += kPrepThreads) {
    const int i = e / d, c = e - i * d;
    const float up = DELTA ? sL[i * ds + c] : log_a * static_cast<float>(i + 1);
    const float end = DELTA ? sL[(n - 1) * ds + c] : log_a * static_cast<float>(n);
    oQg[i * d + c] = sQ[i * ds + c] * expf(up);
    oKe[i * d + c] = sK[i * ds + c] * expf(end - up);
  }
  for (int c = tid; c < d; c += kPrepThreads) oEg[c] = expf(DELTA ? sL[(n - 1) * ds + c] : log_a * static_cast<float>(n));
  if (!DELTA) {
    for (int e = tid; e < n * dv; e += kPrepThreads) {
      const int i = e / dv, c = e - i * dv;
      oUv[i * dv + c] = silu_f(ldf(gv + static_cast<long long>(t0 + i) * p.ld_v + h * dv + c));
    }
    return;
  }
  __syncthreads();  // A is whole; q is no longer needed: its rows become the right-hand sides

  // ---- T X = diag(beta) R by forward substitution, a thread per column, d columns at a time:
  //      first R = K * exp L (X = W), then R = V (X = Uv)
  float* sX = sQ;
  const int n_cols = d + dv;
  for (int c0 = 0; c0 < n_cols; c0 += d) {
    const bool is_w = c0 == 0;
    const int width = is_w ? d : min(d, n_cols - c0);
    for (int c = tid; c < width; c += kPrepThreads) {
      for (int j = 0; j < n; ++j) {
        float r;
        if (is_w) {
          r = sK[j * ds + c] * expf(sL[j * ds + c]);
        } else {
          r = ldf(gv + static_cast<long long>(t0 + j) * p.ld_v + h * dv + (c0 - d) + c);
        }
        const float* arow = sA + j * (kChunk + 1);
        float acc = 0.f;
        for (int m = 0; m < j; ++m) acc += arow[m] * sX[m * ds + c];
        const float x = s_beta[j] * (r - acc);
        sX[j * ds + c] = x;
        if (is_w) oW[j * d + c] = x;
        else oUv[j * dv + (c0 - d) + c] = x;
      }
    }
    // a column is read and written by one thread only: no barrier between the passes
  }
}

// Rows of S owned by a thread in the state update: RPT consecutive rows, d <= 8 * RPT.
template <int RPT, bool DELTA>
__global__ void __launch_bounds__(kApplyThreads)
    chunk_apply_kernel(ChunkArgs p) {
  extern __shared__ __align__(16) float sm[];
  const int d = p.d, dv = p.dv;
  float* sW = sm;                          // [C][d]   (delta)
  float* sKe = sW + (DELTA ? kChunk * d : 0);  // [C][d]
  float* sQg = sKe + kChunk * d;           // [C][d]
  float* sB = sQg + kChunk * d;            // [C][C]
  float* sU = sB + kChunk * kChunk;        // [C][NC]
  float* sS = sU + kChunk * kApplyCols;    // [d][NC]
  float* sEg = sS + d * kApplyCols;        // [d]
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * kApplyCols;
  const int tid = threadIdx.x;
  const int c = tid % kApplyCols, rg = tid / kApplyCols;  // column, row group (8 of them)
  const int first = p.cu[seq], len = p.cu[seq + 1] - first;
  if (len <= 0) return;
  int chunk = 0;
  for (int s = 0; s < seq; ++s) chunk += (p.cu[s + 1] - p.cu[s] + kChunk - 1) / kChunk;
  const bool col_ok = j0 + c < dv;
  float* st = p.state + ((static_cast<size_t>(p.slots[seq]) * p.H + h) * d) * dv;
  for (int e = tid; e < d * kApplyCols; e += kApplyThreads) {
    const int r = e / kApplyCols, cc = e % kApplyCols;
    sS[e] = (j0 + cc < dv) ? st[static_cast<size_t>(r) * dv + j0 + cc] : 0.f;
  }
  const int d4 = d / 4;
  for (int t0 = 0; t0 < len; t0 += kChunk, ++chunk) {
    const int n = min(kChunk, len - t0);
    const size_t ch = static_cast<size_t>(chunk) * p.H + h;
    __syncthreads();  // the chunk before is done with the operands
    {  // operands of this chunk: whole rows, 16 bytes a thread
      const float4* gKe = reinterpret_cast<const float4*>(p.Ke + ch * kChunk * d);
      const float4* gQg = reinterpret_cast<const float4*>(p.Qg + ch * kChunk * d);
      const float4* gW = DELTA ? reinterpret_cast<const float4*>(p.W + ch * kChunk * d) : nullptr;
      for (int e = tid; e < n * d4; e += kApplyThreads) {
        reinterpret_cast<float4*>(sKe)[e] = gKe[e];
        reinterpret_cast<float4*>(sQg)[e] = gQg[e];
        if (DELTA) reinterpret_cast<float4*>(sW)[e] = gW[e];
      }
      const float4* gB = reinterpret_cast<const float4*>(p.B + ch * kChunk * kChunk);
      for (int e = tid; e < n * (kChunk / 4); e += kApplyThreads) reinterpret_cast<float4*>(sB)[e] = gB[e];
      const float* gU = p.Uv + ch * kChunk * dv;
      for (int e = tid; e < n * kApplyCols; e += kApplyThreads) {
        const int i = e / kApplyCols, cc = e % kApplyCols;
        sU[e] = (j0 + cc < dv) ? gU[i * dv + j0 + cc] : 0.f;
      }
      for (int e = tid; e < d; e += kApplyThreads) sEg[e] = p.Eg[ch * d + e];
    }
    __syncthreads();
    // ---- rows i = rg * 8 .. rg * 8 + 7 of U = Uv - W S and of the read-out's first term Qg S
    float o[8], u[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) o[r] = u[r] = 0.f;
    for (int k4 = 0; k4 < d4; ++k4) {
      const float s0 = sS[(4 * k4 + 0) * kApplyCols + c], s1 = sS[(4 * k4 + 1) * kApplyCols + c];
      const float s2 = sS[(4 * k4 + 2) * kApplyCols + c], s3 = sS[(4 * k4 + 3) * kApplyCols + c];
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int i = rg * 8 + r;
        if (i < n) {
          const float4 qv = reinterpret_cast<const float4*>(sQg + i * d)[k4];
          o[r] += qv.x * s0 + qv.y * s1 + qv.z * s2 + qv.w * s3;
          if (DELTA) {
            const float4 wv = reinterpret_cast<const float4*>(sW + i * d)[k4];
            u[r] += wv.x * s0 + wv.y * s1 + wv.z * s2 + wv.w * s3;
          }
        }
      }
    }
    if (DELTA) {
      __syncthreads();  // nobody reads Uv from sU any more (each thread owns its entries, but rows differ below)
#pragma unroll
      for (int r = 0; r < 8; ++r) {
        const int i = rg * 8 + r;
        if (i < n) sU[i * kApplyCols + c] -= u[r];
      }
    }
    __syncthreads();  // U is whole
    // ---- o_i += sum_{j <= i} B_ij u_j, rows out
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int i = rg * 8 + r;
      if (i < n) {
        float acc = o[r];
        const float* brow = sB + i * kChunk;
        for (int j = 0; j <= i; ++j) acc += brow[j] * sU[j * kApplyCols + c];
        if (col_ok) p.out[static_cast<size_t>(first + t0 + i) * (p.H * dv) + h * dv + j0 + c] = acc;
      }
    }
    // ---- S <- diag(Eg) S + Ke^T U: this thread's rows k = rg * RPT .. + RPT - 1 of column c
    float acc[RPT];
#pragma unroll
    for (int r = 0; r < RPT; ++r) acc[r] = 0.f;
    const int k_base = rg * RPT;
    for (int j = 0; j < n; ++j) {
      const float uj = sU[j * kApplyCols + c];
      const float* krow = sKe + j * d + k_base;
#pragma unroll
      for (int r4 = 0; r4 < RPT / 4; ++r4) {
        if (k_base + 4 * r4 < d) {
          const float4 kv = *reinterpret_cast<const float4*>(krow + 4 * r4);
          acc[4 * r4 + 0] += kv.x * uj;
          acc[4 * r4 + 1] += kv.y * uj;
          acc[4 * r4 + 2] += kv.z * uj;
          acc[4 * r4 + 3] += kv.w * uj;
        }
      }
    }
    __syncthreads();  // every thread has read the old S
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int k = k_base + r;
      if (k < d) sS[k * kApplyCols + c] = sEg[k] * sS[k * kApplyCols + c] + acc[r];
    }
  }
  __syncthreads();
  for (int e = tid; e < d * kApplyCols; e += kApplyThreads) {
    const int r = e / kApplyCols, cc = e % kApplyCols;
    if (j0 + cc < dv) st[static_cast<size_t>(r) * dv + j0 + cc] = sS[e];
  }
}

inline size_t prepare_smem(int d, bool delta) {
  return sizeof(float) * (static_cast<size_t>(kChunk) * (d + 1) * (delta ? 3 : 2) + (delta ? kChunk * (kChunk + 1) : 0));
}
inline size_t apply_smem(int d, bool delta) {
  return sizeof(float) * (static_cast<size_t>(kChunk) * d * (delta ? 3 : 2) + kChunk * kChunk + kChunk * kApplyCols +
                          static_cast<size_t>(d) * kApplyCols + d);
}

template <typename S, bool DELTA>
int launch_chunked(const ChunkArgs& a, int n_chunks, cudaStream_t stream) {
  const size_t sp = prepare_smem(a.d, DELTA), sa = apply_smem(a.d, DELTA);
  auto prep = chunk_prepare_kernel<S, DELTA>;
  if (sp > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(prep, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sp));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  launch_pdl(prep, dim3(n_chunks, a.H), dim3(kPrepThreads), sp, stream, a);
  dim3 grid((a.dv + kApplyCols - 1) / kApplyCols, a.H, a.n_seq);
#define PMM_APPLY_CASE(RPT)                                                                                   \
  do {                                                                                                        \
    auto kern = chunk_apply_kernel<RPT, DELTA>;                                                               \
    if (sa > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                           static_cast<int>(sa));                                             \
      if (e != cudaSuccess) return static_cast<int>(e);                                                       \
    }                                                                                                         \
    launch_pdl(kern, grid, dim3(kApplyThreads), sa, stream, a);                                               \
  } while (0)
  if (a.d <= 32) PMM_APPLY_CASE(4);
  else if (a.d <= 64) PMM_APPLY_CASE(8);
  else if (a.d <= 128) PMM_APPLY_CASE(16);
  else PMM_APPLY_CASE(32);
#undef PMM_APPLY_CASE
  return launch_status();
}

}  // namespace pmm

// Whether the chunked kernels take this key size (whole float4 rows, operands of a chunk in one block's
// shared memory).
PMM_EXPORT int pmm_recurrent_chunked_supported(int d, int delta) {
  if (d <= 0 || d % 4) return 0;
  return pmm::prepare_smem(d, delta != 0) <= 220 * 1024 && pmm::apply_smem(d, delta != 0) <= 220 * 1024 ? 1 : 0;
}

// Floats of scratch per (chunk, head).
PMM_EXPORT long long pmm_recurrent_chunked_scratch(int d, int dv, int delta) {
  return static_cast<long long>(pmm::kChunk) * ((delta ? 3 : 2) * d + dv + pmm::kChunk) + d;
}

// n_chunks = sum over sequences of ceil(tokens / 64) (an upper bound is fine: surplus blocks leave).
// scratch: n_chunks * H * pmm_recurrent_chunked_scratch(...) floats, 16-byte aligned.  Other arguments as
// pmm_delta_scan / pmm_decay_scan (decay != nullptr selects the decayed sum).
PMM_EXPORT int pmm_recurrent_chunked(const void* q, long long ld_q, const void* k, long long ld_k, const void* v,
                                     long long ld_v, const void* beta, long long ld_beta, const void* a,
                                     long long ld_a, const float* dt_bias, const float* a_log, const float* decay,
                                     float* state, const int* cu, const int* slots, float* out, float* scratch,
                                     int n_seq, int n_chunks, int H, int Hk, int d, int dv, float unit_eps,
                                     float q_scale, int dtype, cudaStream_t stream) {
  if (n_seq <= 0 || n_chunks <= 0) return 0;
  const bool delta = decay == nullptr;
  if (H <= 0 || Hk <= 0 || H % Hk || dv <= 0 || H > 65535 || n_seq > 65535 || !scratch ||
      reinterpret_cast<uintptr_t>(scratch) % 16 || !pmm_recurrent_chunked_supported(d, delta))
    return PMM_ERR_BAD_ARGUMENT;
  pmm::ChunkArgs p{};
  p.q = q; p.ld_q = ld_q; p.k = k; p.ld_k = ld_k; p.v = v; p.ld_v = ld_v;
  p.beta = beta; p.ld_beta = ld_beta; p.a = a; p.ld_a = ld_a;
  p.dt_bias = dt_bias; p.a_log = a_log; p.decay = decay;
  p.cu = cu; p.n_seq = n_seq; p.H = H; p.Hk = Hk; p.d = d; p.dv = dv;
  p.unit_eps = unit_eps; p.q_scale = q_scale;
  const size_t ch = static_cast<size_t>(n_chunks) * H;
  float* s = scratch;
  // every array starts on a 16-byte boundary: their sizes are multiples of 4 floats except Eg, which is last
  p.Ke = s; s += ch * pmm::kChunk * d;
  p.Qg = s; s += ch * pmm::kChunk * d;
  p.B = s; s += ch * pmm::kChunk * pmm::kChunk;
  if (delta) { p.W = s; s += ch * pmm::kChunk * d; }
  p.Uv = s; s += ch * pmm::kChunk * dv;
  p.Eg = s;
  p.state = state; p.slots = slots; p.out = out;
  PMM_DISPATCH_DTYPE(dtype, S, {
    return delta ? pmm::launch_chunked<S, true>(p, n_chunks, stream) : pmm::launch_chunked<S, false>(p, n_chunks, stream);
  });
  return 0;
}
