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
// the decay.  `chunk_prepare` makes W, Uv, B, Q * exp L, K * exp(L_end - L) and exp L_end for every
// (chunk, head) in parallel.  What follows keeps the chain from chunk to chunk as short as it can be
// and does everything else in parallel over chunks (see the two groups of kernels below): for the
// decayed sum the chain is element-wise, for the delta rule it is one product S <- M S + N per chunk.
// `chunk_apply` is the first, direct form (three products with the state per chunk inside the chain);
// it stays for sizes whose operands the later kernels cannot hold.  All arithmetic is float on the
// CUDA cores: scores, decays, the triangular solve and the state stay 32-bit in both storage types.
// Chunks start at the portion's first token; results do not depend on where a portion is cut beyond
// rounding.
#include "common.cuh"
#include <utility>

namespace pmm {

constexpr int kChunk = 64;
constexpr int kPrepThreads = 512;
constexpr int kApplyThreads = 256;

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
  int sub_blocks;                       // chunk_prepare scales rows once per sub-block of 16 tokens (its shared memory allows it)
  float *N, *M;                         // [d, dv] and (delta) [d, d] per (chunk, head): see the kernels that use them
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

  // ---- A (delta) and B
  if (DELTA && p.sub_blocks) {
    // Pairs inside one sub-block of 16 tokens: the exponential per channel.  A warp takes two rows,
    // 16 lanes each, a lane one column of the row's sub-block.
    for (int i2 = 2 * warp; i2 < n; i2 += 2 * (kPrepThreads / 32)) {
      const int i = i2 + (lane >> 4), j = (i & ~15) + (lane & 15);
      if (i < n && j <= i) {
        const float *qi = sQ + i * ds, *ki = sK + i * ds, *li = sL + i * ds, *kj = sK + j * ds, *lj = sL + j * ds;
        float accA = 0.f, accB = 0.f;
        for (int c = 0; c < d; ++c) {
          const float w = expf(li[c] - lj[c]) * kj[c];
          accA += ki[c] * w;
          accB += qi[c] * w;
        }
        sA[i * (kChunk + 1) + j] = accA;
        oB[i * kChunk + j] = accB;
      }
    }
    // Pairs across sub-blocks: with r the last row before i's sub-block, exp(L_i - L_j) = exp(L_i - L_r) exp(L_r - L_j),
    // both factors at most one, so the rows are scaled once per sub-block and the pairs are plain dot products.
    float* sKd = sA + kChunk * (kChunk + 1);   // [48][ds]  k_j exp(L_r - L_j), j before the sub-block
    float* sKp = sKd + 48 * ds;                // [16][ds]  k_i exp(L_i - L_r), i in the sub-block
    float* sQp = sKp + 16 * ds;                // [16][ds]  q_i exp(L_i - L_r)
    for (int blk = 1; 16 * blk < n; ++blk) {
      const int r = 16 * blk - 1, rows = min(16, n - 16 * blk);
      __syncthreads();  // the sub-block before is done with the scaled rows
      for (int e = tid; e < 16 * blk * d; e += kPrepThreads) {
        const int j = e / d, c = e - j * d;
        sKd[j * ds + c] = sK[j * ds + c] * expf(sL[r * ds + c] - sL[j * ds + c]);
      }
      for (int e = tid; e < rows * d; e += kPrepThreads) {
        const int ii = e / d, c = e - ii * d, i = 16 * blk + ii;
        const float pw = expf(sL[i * ds + c] - sL[r * ds + c]);
        sKp[ii * ds + c] = sK[i * ds + c] * pw;
        sQp[ii * ds + c] = sQ[i * ds + c] * pw;
      }
      __syncthreads();
      if (warp < rows) {  // a warp per row of the sub-block, a lane the columns j = lane and lane + 32
        const int i = 16 * blk + warp;
        const float *kp = sKp + warp * ds, *qp = sQp + warp * ds;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int j = lane + 32 * half;
          if (j < 16 * blk) {
            const float* kd = sKd + j * ds;
            float accA = 0.f, accB = 0.f;
            for (int c = 0; c < d; ++c) {
              accA += kp[c] * kd[c];
              accB += qp[c] * kd[c];
            }
            sA[i * (kChunk + 1) + j] = accA;
            oB[i * kChunk + j] = accB;
          }
        }
      }
    }
  } else {
  // a warp takes rows i, a lane the columns j = lane and lane + 32
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

  // ---- T X = diag(beta) R by forward substitution in place, a thread per column.  R = K * exp L
  //      (X = W) lies where q was; R = V (X = Uv), d columns at a time, where the logarithms were:
  //      they are no longer needed once K * exp L is made.
  float* sXw = sQ;
  float* sXv = sL;
  for (int e = tid; e < n * d; e += kPrepThreads) {
    const int i = e / d, c = e - i * d;
    sXw[i * ds + c] = sK[i * ds + c] * expf(sL[i * ds + c]);
  }
  __syncthreads();
  for (int v0 = 0; v0 < dv; v0 += d) {
    const int vw = min(d, dv - v0);
    for (int e = tid; e < n * vw; e += kPrepThreads) {
      const int i = e / vw, c = e - i * vw;
      sXv[i * ds + c] = ldf(gv + static_cast<long long>(t0 + i) * p.ld_v + h * dv + v0 + c);
    }
    __syncthreads();
    const int n_cols = (v0 == 0 ? d : 0) + vw;  // the first pass also solves for W
    for (int col = tid; col < n_cols; col += kPrepThreads) {
      const bool is_w = v0 == 0 && col < d;
      const int c = is_w ? col : col - (v0 == 0 ? d : 0);
      float* x = (is_w ? sXw : sXv) + c;
      for (int j = 0; j < n; ++j) {
        const float* arow = sA + j * (kChunk + 1);
        float acc0 = 0.f, acc1 = 0.f;
        int m = 0;
        for (; m + 1 < j; m += 2) {
          acc0 += arow[m] * x[m * ds];
          acc1 += arow[m + 1] * x[(m + 1) * ds];
        }
        if (m < j) acc0 += arow[m] * x[m * ds];
        const float xj = s_beta[j] * (x[j * ds] - (acc0 + acc1));
        x[j * ds] = xj;
        if (is_w) oW[j * d + c] = xj;
        else oUv[j * dv + v0 + c] = xj;
      }
    }
    __syncthreads();  // the next pass loads further columns of V over these
  }
}

__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src) {
  const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }

// A block owns NC (16, or 8 where that is needed to fill the GPU) columns of one head's state for one
// sequence and walks the sequence's chunks in order.  Thread (column c, row group rg of 256 / NC): rows
// rg * NC/4 .. of the chunk in the products with S, rows rg * RPT .. + RPT - 1 of S in the state update
// (d <= RPT * 256 / NC).  The next chunk's
// operands come by asynchronous copies while this chunk is computed: Q * exp L and W as soon as the
// products with S are done, B, K * exp(L_end - L) and Uv once the state update has read them.
template <int NC, int RPT, bool DELTA>
__global__ void __launch_bounds__(kApplyThreads)
    chunk_apply_kernel(ChunkArgs p) {
  constexpr int kRows = kChunk / (kApplyThreads / NC);  // rows of a chunk per thread in the products with S
  extern __shared__ __align__(16) float sm[];
  const int d = p.d, dv = p.dv;
  float* sW = sm;                          // [C][d]   (delta)
  float* sKe = sW + (DELTA ? kChunk * d : 0);  // [C][d]
  float* sQg = sKe + kChunk * d;           // [C][d]
  float* sB = sQg + kChunk * d;            // [C][C]
  float* sU = sB + kChunk * kChunk;        // [C][NC]
  float* sS = sU + kChunk * NC;    // [d][NC]
  float* sEg = sS + d * NC;        // [d]
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * NC;
  const int tid = threadIdx.x;
  const int c = tid % NC, rg = tid / NC;
  const int first = p.cu[seq], len = p.cu[seq + 1] - first;
  if (len <= 0) return;
  int chunk0 = 0;
  for (int s = 0; s < seq; ++s) chunk0 += (p.cu[s + 1] - p.cu[s] + kChunk - 1) / kChunk;
  const bool col_ok = j0 + c < dv;
  const bool tile_async = dv % 4 == 0;
  const int d4 = d / 4;
  float* st = p.state + ((static_cast<size_t>(p.slots[seq]) * p.H + h) * d) * dv;

  auto fetch_early = [&](int chunk, int n) {   // operands of the products with S
    const size_t ch = static_cast<size_t>(chunk) * p.H + h;
    const float* gQg = p.Qg + ch * kChunk * d;
    for (int e = tid; e < n * d4; e += kApplyThreads) cp_async16(sQg + 4 * e, gQg + 4 * e);
    if (DELTA) {
      const float* gW = p.W + ch * kChunk * d;
      for (int e = tid; e < n * d4; e += kApplyThreads) cp_async16(sW + 4 * e, gW + 4 * e);
    }
    cp_async_commit();
  };
  auto fetch_late = [&](int chunk, int n) {    // the rest
    const size_t ch = static_cast<size_t>(chunk) * p.H + h;
    const float* gKe = p.Ke + ch * kChunk * d;
    for (int e = tid; e < n * d4; e += kApplyThreads) cp_async16(sKe + 4 * e, gKe + 4 * e);
    const float* gB = p.B + ch * kChunk * kChunk;
    for (int e = tid; e < n * (kChunk / 4); e += kApplyThreads) cp_async16(sB + 4 * e, gB + 4 * e);
    const float* gU = p.Uv + ch * kChunk * dv;
    if (tile_async) {
      for (int e = tid; e < n * (NC / 4); e += kApplyThreads) {
        const int i = e / (NC / 4), g = e % (NC / 4);
        if (j0 + 4 * g < dv) cp_async16(sU + i * NC + 4 * g, gU + static_cast<size_t>(i) * dv + j0 + 4 * g);
        else *reinterpret_cast<float4*>(sU + i * NC + 4 * g) = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
      for (int e = tid; e < n * NC; e += kApplyThreads) {
        const int i = e / NC, cc = e % NC;
        sU[e] = (j0 + cc < dv) ? gU[static_cast<size_t>(i) * dv + j0 + cc] : 0.f;
      }
    }
    for (int e = tid; e < d4; e += kApplyThreads) cp_async16(sEg + 4 * e, p.Eg + ch * d + 4 * e);
    cp_async_commit();
  };

  fetch_early(chunk0, min(kChunk, len));
  fetch_late(chunk0, min(kChunk, len));
  for (int e = tid; e < d * NC; e += kApplyThreads) {
    const int r = e / NC, cc = e % NC;
    sS[e] = (j0 + cc < dv) ? st[static_cast<size_t>(r) * dv + j0 + cc] : 0.f;
  }
  int chunk = chunk0;
  for (int t0 = 0; t0 < len; t0 += kChunk, ++chunk) {
    const int n = min(kChunk, len - t0);
    const bool more = t0 + kChunk < len;
    const int n_next = more ? min(kChunk, len - t0 - kChunk) : 0;
    cp_async_wait<1>();  // Q * exp L and W of this chunk have landed (the later group may still fly)
    __syncthreads();     // ... for every thread, and everyone's rows of S are written
    // ---- rows i = rg * 4 .. + 3 of W S and of the read-out's first term (Q * exp L) S
    float o[kRows], u[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) o[r] = u[r] = 0.f;
    for (int k4 = 0; k4 < d4; ++k4) {
      const float s0 = sS[(4 * k4 + 0) * NC + c], s1 = sS[(4 * k4 + 1) * NC + c];
      const float s2 = sS[(4 * k4 + 2) * NC + c], s3 = sS[(4 * k4 + 3) * NC + c];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const int i = rg * kRows + r;
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
    cp_async_wait<0>();  // B, K * exp(L_end - L) and Uv
    __syncthreads();     // ... for every thread; everyone is done with Q * exp L and W
    if (more) fetch_early(chunk + 1, n_next);
    if (DELTA) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const int i = rg * kRows + r;
        if (i < n) sU[i * NC + c] -= u[r];  // U = Uv - W S
      }
      __syncthreads();  // U is whole
    }
    // ---- o_i += sum_{j <= i} B_ij u_j, rows out
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const int i = rg * kRows + r;
      if (i < n) {
        float acc = o[r];
        const float* brow = sB + i * kChunk;
        for (int j = 0; j <= i; ++j) acc += brow[j] * sU[j * NC + c];
        if (col_ok) p.out[static_cast<size_t>(first + t0 + i) * (p.H * dv) + h * dv + j0 + c] = acc;
      }
    }
    // ---- S <- diag(exp L_end) S + (K * exp(L_end - L))^T U: rows k = rg * RPT .. + RPT - 1 of column c
    float acc[RPT];
#pragma unroll
    for (int r = 0; r < RPT; ++r) acc[r] = 0.f;
    const int k_base = rg * RPT;
    for (int j = 0; j < n; ++j) {
      const float uj = sU[j * NC + c];
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
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int k = k_base + r;
      if (k < d) sS[k * NC + c] = sEg[k] * sS[k * NC + c] + acc[r];  // own entries only
    }
    __syncthreads();  // everyone is done with B, K * exp(L_end - L), U and exp L_end
    if (more) fetch_late(chunk + 1, n_next);
    else cp_async_commit();  // keeps the count of groups in flight the same on the last round
  }
  cp_async_wait<0>();
  __syncthreads();
  for (int e = tid; e < d * NC; e += kApplyThreads) {
    const int r = e / NC, cc = e % NC;
    if (j0 + cc < dv) st[static_cast<size_t>(r) * dv + j0 + cc] = sS[e];
  }
}

// ----------------------------------------------------------------------------------------------
// The decayed sum has no product with the state inside its chain: S_end = a^n S_0 + N with
// N = (K * a^(n-1-j))^T V, so the chain over a sequence's chunks is element-wise.  Three launches after
// chunk_prepare, all but the middle one parallel over chunks: (1) N of every chunk; (2) a running
// pass per state element that leaves every chunk's starting state where its N was; (3) the rows
// o_i = (q_i a^(i+1))^T S_0 + sum_{j<=i} B_ij v_j of every chunk.
constexpr int kDecayTile = 64;      // state columns per block in (1) and (3)
constexpr int kDecayThreads = 256;

// ---- small products on shared-memory operands, 4 x 4 results a thread (16 multiply-adds per two
// 16-byte loads).  Tiles are 64 columns wide; thread t of 256 owns columns 4 (t % 16) .. + 3.
__device__ __forceinline__ void fma4x4(float (&acc)[4][4], const float4& a, const float4& b) {
  const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] += av[r] * bv[c];
}

// acc[r][c] = sum_{j < n} A[j][k0 + r] * R[j][c0 + c]   (A rows of stride lda, R rows of stride 64)
__device__ __forceinline__ void product_tn(float (&acc)[4][4], const float* __restrict__ A, int lda, int k0,
                                           const float* __restrict__ R, int c0, int n) {
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
  for (int j = 0; j < n; ++j)
    fma4x4(acc, *reinterpret_cast<const float4*>(A + j * lda + k0), *reinterpret_cast<const float4*>(R + j * kDecayTile + c0));
}

// acc[r][c] += sum_{k < kn} A[i0 + r][k] * R[k][c0 + c], kn a multiple of 4; with `tri`, only k <= i0 + r
__device__ __forceinline__ void product_nn(float (&acc)[4][4], const float* __restrict__ A, int lda, int i0,
                                           const float* __restrict__ R, int c0, int kn, bool tri) {
  for (int k4 = 0; k4 < kn; k4 += 4) {
    float4 a[4], b[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) a[r] = *reinterpret_cast<const float4*>(A + (i0 + r) * lda + k4);
#pragma unroll
    for (int q = 0; q < 4; ++q) b[q] = *reinterpret_cast<const float4*>(R + (k4 + q) * kDecayTile + c0);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float av[4] = {a[r].x, a[r].y, a[r].z, a[r].w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (!tri || k4 + q <= i0 + r) {
          acc[r][0] += av[q] * b[q].x;
          acc[r][1] += av[q] * b[q].y;
          acc[r][2] += av[q] * b[q].z;
          acc[r][3] += av[q] * b[q].w;
        }
      }
    }
  }
}

// N [d, dv] per (chunk, head), chunk-major
__global__ void __launch_bounds__(kDecayThreads)
    decay_chunk_state_kernel(ChunkArgs p) {
  extern __shared__ __align__(16) float sm[];
  const int d = p.d, dv = p.dv;
  float* sKe = sm;                    // [C][d]
  float* sV = sKe + kChunk * d;       // [C][tile]
  pdl_launch_dependents();
  pdl_wait();
  const int chunk = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * kDecayTile;
  int seq, t0, n;
  if (!locate_chunk(p.cu, p.n_seq, chunk, &seq, &t0, &n)) return;
  const int tid = threadIdx.x;
  const size_t ch = static_cast<size_t>(chunk) * p.H + h;
  const float* gKe = p.Ke + ch * kChunk * d;
  const float* gV = p.Uv + ch * kChunk * dv;
  for (int e = tid; e < n * d; e += kDecayThreads) sKe[e] = gKe[e];
  for (int e = tid; e < n * kDecayTile; e += kDecayThreads) {
    const int j = e / kDecayTile, c = e % kDecayTile;
    sV[e] = (c0 + c < dv) ? gV[static_cast<size_t>(j) * dv + c0 + c] : 0.f;
  }
  __syncthreads();
  float* gN = p.N + ch * static_cast<size_t>(d) * dv;
  const int cc = 4 * (tid % 16);
  for (int k0 = 4 * (tid / 16); k0 < d; k0 += 4 * (kDecayThreads / 16)) {
    float acc[4][4];
    product_tn(acc, sKe, d, k0, sV, cc, n);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (c0 + cc + c < dv) gN[static_cast<size_t>(k0 + r) * dv + c0 + cc + c] = acc[r][c];
  }
}

// per state element: S_0 of every chunk replaces its N; the request's state moves to the end of the portion
__global__ void __launch_bounds__(kDecayThreads)
    decay_chunk_scan_kernel(ChunkArgs p) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y;
  const int d = p.d, dv = p.dv;
  const int e = blockIdx.x * kDecayThreads + threadIdx.x;
  if (e >= d * dv) return;
  const int first = p.cu[seq], len = p.cu[seq + 1] - first;
  if (len <= 0) return;
  int chunk = 0;
  for (int s = 0; s < seq; ++s) chunk += (p.cu[s + 1] - p.cu[s] + kChunk - 1) / kChunk;
  const int k = e / dv;
  float* st = p.state + (static_cast<size_t>(p.slots[seq]) * p.H + h) * d * dv + e;
  float s = *st;
  const int n_chunks = (len + kChunk - 1) / kChunk;
  constexpr int kAhead = 8;  // the chain is one multiply-add a chunk: the loads are what takes time, so 8 fly at once
  for (int c0 = 0; c0 < n_chunks; c0 += kAhead) {
    float add[kAhead], eg[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (c0 + u < n_chunks) {
        const size_t ch = static_cast<size_t>(chunk + c0 + u) * p.H + h;
        add[u] = p.N[ch * static_cast<size_t>(d) * dv + e];
        eg[u] = p.Eg[ch * d + k];
      }
    }
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (c0 + u < n_chunks) {
        const size_t ch = static_cast<size_t>(chunk + c0 + u) * p.H + h;
        p.N[ch * static_cast<size_t>(d) * dv + e] = s;
        s = eg[u] * s + add[u];
      }
    }
  }
  *st = s;
}

__global__ void __launch_bounds__(kDecayThreads)
    decay_chunk_output_kernel(ChunkArgs p) {
  extern __shared__ __align__(16) float sm[];
  const int d = p.d, dv = p.dv;
  float* sQg = sm;                          // [C][d]
  float* sB = sQg + kChunk * d;             // [C][C]
  float* sS = sB + kChunk * kChunk;         // [d][tile]
  float* sV = sS + d * kDecayTile;          // [C][tile]
  pdl_launch_dependents();
  pdl_wait();
  const int chunk = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * kDecayTile;
  int seq, t0, n;
  if (!locate_chunk(p.cu, p.n_seq, chunk, &seq, &t0, &n)) return;
  const int tid = threadIdx.x;
  const size_t ch = static_cast<size_t>(chunk) * p.H + h;
  const float* gQg = p.Qg + ch * kChunk * d;
  const float* gB = p.B + ch * kChunk * kChunk;
  const float* gS = p.N + ch * static_cast<size_t>(d) * dv;
  const float* gV = p.Uv + ch * kChunk * dv;
  for (int e = tid; e < n * d; e += kDecayThreads) sQg[e] = gQg[e];
  for (int e = tid; e < n * kChunk; e += kDecayThreads) sB[e] = gB[e];
  for (int e = tid; e < d * kDecayTile; e += kDecayThreads) {
    const int k = e / kDecayTile, c = e % kDecayTile;
    sS[e] = (c0 + c < dv) ? gS[static_cast<size_t>(k) * dv + c0 + c] : 0.f;
  }
  for (int e = tid; e < n * kDecayTile; e += kDecayThreads) {
    const int j = e / kDecayTile, c = e % kDecayTile;
    sV[e] = (c0 + c < dv) ? gV[static_cast<size_t>(j) * dv + c0 + c] : 0.f;
  }
  __syncthreads();
  // thread: rows i0 .. i0 + 3, columns cc .. cc + 3 (rows at and beyond n hold stale values that are not stored)
  const int cc = 4 * (tid % 16), i0 = 4 * (tid / 16);
  if (i0 < n) {
    float acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
    product_nn(acc, sQg, d, i0, sS, cc, d, false);
    product_nn(acc, sB, kChunk, i0, sV, cc, i0 + 4, true);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (i0 + r < n && c0 + cc + c < dv)
          p.out[static_cast<size_t>(t0 + i0 + r) * (p.H * dv) + h * dv + c0 + cc + c] = acc[r][c];
  }
}

// ----------------------------------------------------------------------------------------------
// The delta rule's link from chunk to chunk, S_end = diag(exp L_end) S_0 + Ke^T (Uv - W S_0) with
// Ke = K * exp(L_end - L), is one product with the state once it is written as
//   S_end = M S_0 + N,    M = diag(exp L_end) - Ke^T W  [d, d],    N = Ke^T Uv  [d, dv],
// and M and N do not depend on the state.  Three launches after chunk_prepare: (1) M and N of every
// chunk in parallel; (2) the chain, a block per (sequence, head, 8 state columns), one product a chunk,
// the next chunk's M fetched meanwhile, every chunk's starting state left where its N was; (3) the
// rows o_i = (q_i * exp L_i)^T S_0 + sum_{j<=i} B_ij u_j, U = Uv - W S_0, of every chunk in parallel.
constexpr int kChainCols = 8;

// X = Ke^T [-W | Uv]: columns below d go to M (with exp L_end on the diagonal), the others to N
__global__ void __launch_bounds__(kDecayThreads)
    delta_chunk_compose_kernel(ChunkArgs p, float* __restrict__ gM_all) {
  extern __shared__ __align__(16) float sm[];
  const int d = p.d, dv = p.dv;
  float* sKe = sm;                    // [C][d]
  float* sR = sKe + kChunk * d;       // [C][tile]
  pdl_launch_dependents();
  pdl_wait();
  const int chunk = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * kDecayTile;
  int seq, t0, n;
  if (!locate_chunk(p.cu, p.n_seq, chunk, &seq, &t0, &n)) return;
  const int tid = threadIdx.x;
  const size_t ch = static_cast<size_t>(chunk) * p.H + h;
  const float* gKe = p.Ke + ch * kChunk * d;
  const float* gW = p.W + ch * kChunk * d;
  const float* gUv = p.Uv + ch * kChunk * dv;
  for (int e = tid; e < n * d; e += kDecayThreads) sKe[e] = gKe[e];
  for (int e = tid; e < n * kDecayTile; e += kDecayThreads) {
    const int j = e / kDecayTile, col = c0 + e % kDecayTile;
    float v = 0.f;
    if (col < d) v = -gW[static_cast<size_t>(j) * d + col];
    else if (col < d + dv) v = gUv[static_cast<size_t>(j) * dv + col - d];
    sR[e] = v;
  }
  __syncthreads();
  float* gM = gM_all + ch * static_cast<size_t>(d) * d;
  float* gN = p.N + ch * static_cast<size_t>(d) * dv;
  const int cc = 4 * (tid % 16);
  for (int k0 = 4 * (tid / 16); k0 < d; k0 += 4 * (kDecayThreads / 16)) {
    float acc[4][4];
    product_tn(acc, sKe, d, k0, sR, cc, n);
#pragma unroll
    for (int r = 0; r < 4; ++r) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int k = k0 + r, col = c0 + cc + c;
        if (col < d) gM[static_cast<size_t>(k) * d + col] = acc[r][c] + (k == col ? p.Eg[ch * d + k] : 0.f);
        else if (col < d + dv) gN[static_cast<size_t>(k) * dv + col - d] = acc[r][c];
      }
    }
  }
}

template <int RPT>  // rows of S per thread: d <= 32 * RPT
__global__ void __launch_bounds__(kDecayThreads)
    delta_chunk_chain_kernel(ChunkArgs p, const float* __restrict__ gM_all, int n_buf) {
  extern __shared__ __align__(16) float sm[];
  const int d = p.d, dv = p.dv;
  float* sM = sm;                                   // [n_buf][d][d]
  float* sS = sM + static_cast<size_t>(n_buf) * d * d;  // [d][NC]
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * kChainCols;
  const int tid = threadIdx.x;
  const int c = tid % kChainCols, kg = tid / kChainCols;  // 32 row groups
  const int first = p.cu[seq], len = p.cu[seq + 1] - first;
  if (len <= 0) return;
  int chunk0 = 0;
  for (int s = 0; s < seq; ++s) chunk0 += (p.cu[s + 1] - p.cu[s] + kChunk - 1) / kChunk;
  const int n_chunks = (len + kChunk - 1) / kChunk;
  const bool col_ok = j0 + c < dv;
  const int dd4 = d * d / 4, d4 = d / 4;
  float* st = p.state + ((static_cast<size_t>(p.slots[seq]) * p.H + h) * d) * dv;
  auto fetch = [&](int ci) {
    const float* gM = gM_all + (static_cast<size_t>(chunk0 + ci) * p.H + h) * static_cast<size_t>(d) * d;
    float* dst = sM + static_cast<size_t>(ci % n_buf) * d * d;
    for (int e = tid; e < dd4; e += kDecayThreads) cp_async16(dst + 4 * e, gM + 4 * e);
    cp_async_commit();
  };
  fetch(0);
  for (int e = tid; e < d * kChainCols; e += kDecayThreads) {
    const int r = e / kChainCols, cc = e % kChainCols;
    sS[e] = (j0 + cc < dv) ? st[static_cast<size_t>(r) * dv + j0 + cc] : 0.f;
  }
  for (int ci = 0; ci < n_chunks; ++ci) {
    if (n_buf > 1 && ci + 1 < n_chunks) {
      fetch(ci + 1);        // into the other buffer, whose product ended before the barrier below
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();        // M of this chunk and everyone's rows of S are there
    const float* M = sM + static_cast<size_t>(ci % n_buf) * d * d;
    float* gN = p.N + (static_cast<size_t>(chunk0 + ci) * p.H + h) * static_cast<size_t>(d) * dv;
    float acc[RPT], nv[RPT];
#pragma unroll
    for (int r = 0; r < RPT; ++r) {  // N comes from global memory while the product runs
      const int k = kg + 32 * r;
      nv[r] = (k < d && col_ok) ? gN[static_cast<size_t>(k) * dv + j0 + c] : 0.f;
      acc[r] = 0.f;
    }
    for (int q4 = 0; q4 < d4; ++q4) {
      const float s0 = sS[(4 * q4 + 0) * kChainCols + c], s1 = sS[(4 * q4 + 1) * kChainCols + c];
      const float s2 = sS[(4 * q4 + 2) * kChainCols + c], s3 = sS[(4 * q4 + 3) * kChainCols + c];
#pragma unroll
      for (int r = 0; r < RPT; ++r) {
        const int k = kg + 32 * r;
        if (k < d) {
          const float4 m = reinterpret_cast<const float4*>(M + static_cast<size_t>(k) * d)[q4];
          acc[r] += m.x * s0 + m.y * s1 + m.z * s2 + m.w * s3;
        }
      }
    }
    __syncthreads();        // everyone has read S (and this chunk's M)
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      const int k = kg + 32 * r;
      if (k < d) {
        if (col_ok) gN[static_cast<size_t>(k) * dv + j0 + c] = sS[k * kChainCols + c];  // the chunk's starting state
        sS[k * kChainCols + c] = acc[r] + nv[r];
      }
    }
    if (n_buf == 1 && ci + 1 < n_chunks) fetch(ci + 1);
  }
  __syncthreads();
  for (int e = tid; e < d * kChainCols; e += kDecayThreads) {
    const int r = e / kChainCols, cc = e % kChainCols;
    if (j0 + cc < dv) st[static_cast<size_t>(r) * dv + j0 + cc] = sS[e];
  }
}

__global__ void __launch_bounds__(kDecayThreads)
    delta_chunk_output_kernel(ChunkArgs p) {
  extern __shared__ __align__(16) float sm[];
  const int d = p.d, dv = p.dv;
  float* sQg = sm;                          // [C][d]
  float* sW = sQg + kChunk * d;             // [C][d]
  float* sB = sW + kChunk * d;              // [C][C]
  float* sS = sB + kChunk * kChunk;         // [d][tile]
  float* sU = sS + d * kDecayTile;          // [C][tile]
  pdl_launch_dependents();
  pdl_wait();
  const int chunk = blockIdx.x, h = blockIdx.y, c0 = blockIdx.z * kDecayTile;
  int seq, t0, n;
  if (!locate_chunk(p.cu, p.n_seq, chunk, &seq, &t0, &n)) return;
  const int tid = threadIdx.x;
  const size_t ch = static_cast<size_t>(chunk) * p.H + h;
  const float* gQg = p.Qg + ch * kChunk * d;
  const float* gW = p.W + ch * kChunk * d;
  const float* gB = p.B + ch * kChunk * kChunk;
  const float* gS = p.N + ch * static_cast<size_t>(d) * dv;
  const float* gUv = p.Uv + ch * kChunk * dv;
  const int d4 = d / 4;
  for (int e = tid; e < n * d4; e += kDecayThreads) {
    reinterpret_cast<float4*>(sQg)[e] = reinterpret_cast<const float4*>(gQg)[e];
    reinterpret_cast<float4*>(sW)[e] = reinterpret_cast<const float4*>(gW)[e];
  }
  for (int e = tid; e < n * kChunk; e += kDecayThreads) sB[e] = gB[e];
  for (int e = tid; e < d * kDecayTile; e += kDecayThreads) {
    const int k = e / kDecayTile, c = e % kDecayTile;
    sS[e] = (c0 + c < dv) ? gS[static_cast<size_t>(k) * dv + c0 + c] : 0.f;
  }
  for (int e = tid; e < n * kDecayTile; e += kDecayThreads) {
    const int j = e / kDecayTile, c = e % kDecayTile;
    sU[e] = (c0 + c < dv) ? gUv[static_cast<size_t>(j) * dv + c0 + c] : 0.f;
  }
  __syncthreads();
  // thread: rows i0 .. i0 + 3, columns cc .. cc + 3
  const int cc = 4 * (tid % 16), i0 = 4 * (tid / 16);
  float o[4][4], u[4][4];
#pragma unroll
  for (int r = 0; r < 4; ++r)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[r][c] = u[r][c] = 0.f;
  if (i0 < n) {
    product_nn(o, sQg, d, i0, sS, cc, d, false);
    product_nn(u, sW, d, i0, sS, cc, d, false);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c) sU[(i0 + r) * kDecayTile + cc + c] -= u[r][c];  // U = Uv - W S_0 (own entries)
  }
  __syncthreads();
  if (i0 < n) {
    product_nn(o, sB, kChunk, i0, sU, cc, i0 + 4, true);
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
      for (int c = 0; c < 4; ++c)
        if (i0 + r < n && c0 + cc + c < dv)
          p.out[static_cast<size_t>(t0 + i0 + r) * (p.H * dv) + h * dv + c0 + cc + c] = o[r][c];
  }
}

inline size_t prepare_smem(int d, bool delta, bool sub_blocks = false) {
  return sizeof(float) * (static_cast<size_t>(kChunk) * (d + 1) * (delta ? 3 : 2) + (delta ? kChunk * (kChunk + 1) : 0) +
                          (sub_blocks ? static_cast<size_t>(48 + 32) * (d + 1) : 0));
}
inline size_t apply_smem(int d, bool delta, int nc = 16) {
  return sizeof(float) * (static_cast<size_t>(kChunk) * d * (delta ? 3 : 2) + kChunk * kChunk + kChunk * nc +
                          static_cast<size_t>(d) * nc + d);
}

template <typename S, bool DELTA>
int launch_chunked(ChunkArgs a, int n_chunks, cudaStream_t stream) {
  a.sub_blocks = DELTA && prepare_smem(a.d, true, true) <= 220 * 1024;
  const size_t sp = prepare_smem(a.d, DELTA, a.sub_blocks != 0);
  auto prep = chunk_prepare_kernel<S, DELTA>;
  if (sp > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(prep, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(sp));
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  launch_pdl(prep, dim3(n_chunks, a.H), dim3(kPrepThreads), sp, stream, a);
  if (DELTA) {
    const int d = a.d;
    const int tiles_c = (d + a.dv + kDecayTile - 1) / kDecayTile, tiles_o = (a.dv + kDecayTile - 1) / kDecayTile;
    const size_t s1 = sizeof(float) * kChunk * (static_cast<size_t>(d) + kDecayTile);
    const size_t m_bytes = sizeof(float) * static_cast<size_t>(d) * d, s_bytes = sizeof(float) * d * kChainCols;
    const int n_buf = 2 * m_bytes + s_bytes <= 200 * 1024 ? 2 : 1;
    const size_t s2 = n_buf * m_bytes + s_bytes;
    const size_t s3 = sizeof(float) * (2 * static_cast<size_t>(kChunk) * d + kChunk * kChunk +
                                       static_cast<size_t>(d) * kDecayTile + kChunk * kDecayTile);
    if (s2 <= 200 * 1024 && s3 <= 200 * 1024) {
      auto chain = d <= 64 ? delta_chunk_chain_kernel<2> : d <= 128 ? delta_chunk_chain_kernel<4> : delta_chunk_chain_kernel<8>;
      cudaError_t e = cudaSuccess;
      if (s1 > 48 * 1024) e = cudaFuncSetAttribute(delta_chunk_compose_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(s1));
      if (e == cudaSuccess && s2 > 48 * 1024) e = cudaFuncSetAttribute(chain, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(s2));
      if (e == cudaSuccess && s3 > 48 * 1024) e = cudaFuncSetAttribute(delta_chunk_output_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(s3));
      if (e != cudaSuccess) return static_cast<int>(e);
      launch_pdl(delta_chunk_compose_kernel, dim3(n_chunks, a.H, tiles_c), dim3(kDecayThreads), s1, stream, a, a.M);
      launch_pdl(chain, dim3((a.dv + kChainCols - 1) / kChainCols, a.H, a.n_seq), dim3(kDecayThreads), s2, stream, a,
                 static_cast<const float*>(a.M), n_buf);
      launch_pdl(delta_chunk_output_kernel, dim3(n_chunks, a.H, tiles_o), dim3(kDecayThreads), s3, stream, a);
      return launch_status();
    }
  }
  if (!DELTA) {
    const int tiles = (a.dv + kDecayTile - 1) / kDecayTile;
    const size_t s1 = sizeof(float) * kChunk * (static_cast<size_t>(a.d) + kDecayTile);
    const size_t s3 = sizeof(float) * (static_cast<size_t>(kChunk) * a.d + kChunk * kChunk +
                                       static_cast<size_t>(a.d) * kDecayTile + kChunk * kDecayTile);
    if (s3 <= 200 * 1024 && tiles <= 65535) {
      for (auto pair : {std::make_pair(decay_chunk_state_kernel, s1), std::make_pair(decay_chunk_output_kernel, s3)}) {
        if (pair.second > 48 * 1024) {
          cudaError_t e = cudaFuncSetAttribute(pair.first, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               static_cast<int>(pair.second));
          if (e != cudaSuccess) return static_cast<int>(e);
        }
      }
      launch_pdl(decay_chunk_state_kernel, dim3(n_chunks, a.H, tiles), dim3(kDecayThreads), s1, stream, a);
      launch_pdl(decay_chunk_scan_kernel, dim3((a.d * a.dv + kDecayThreads - 1) / kDecayThreads, a.H, a.n_seq),
                 dim3(kDecayThreads), 0, stream, a);
      launch_pdl(decay_chunk_output_kernel, dim3(n_chunks, a.H, tiles), dim3(kDecayThreads), s3, stream, a);
      return launch_status();
    }
  }
  // 16 state columns a block; 8 where 16 would leave most of the GPU without a block
  const bool narrow = static_cast<long long>((a.dv + 15) / 16) * a.H * a.n_seq < 100;
  const int nc = narrow ? 8 : 16;
  const size_t sa = apply_smem(a.d, DELTA, nc);
  dim3 grid((a.dv + nc - 1) / nc, a.H, a.n_seq);
#define PMM_APPLY_CASE(NC, RPT)                                                                               \
  do {                                                                                                        \
    auto kern = chunk_apply_kernel<NC, RPT, DELTA>;                                                           \
    if (sa > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,                 \
                                           static_cast<int>(sa));                                             \
      if (e != cudaSuccess) return static_cast<int>(e);                                                       \
    }                                                                                                         \
    launch_pdl(kern, grid, dim3(kApplyThreads), sa, stream, a);                                               \
  } while (0)
  if (narrow) {
    if (a.d <= 128) PMM_APPLY_CASE(8, 4);
    else PMM_APPLY_CASE(8, 8);
  } else {
    if (a.d <= 64) PMM_APPLY_CASE(16, 4);
    else if (a.d <= 128) PMM_APPLY_CASE(16, 8);
    else if (a.d <= 192) PMM_APPLY_CASE(16, 12);
    else PMM_APPLY_CASE(16, 16);
  }
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
  // Ke, Qg, Uv, B, Eg; N (then every chunk's starting state); for the delta rule also W and M
  const long long w = delta ? static_cast<long long>(pmm::kChunk) * d + static_cast<long long>(d) * d : 0;
  return static_cast<long long>(pmm::kChunk) * (2 * d + dv + pmm::kChunk) + static_cast<long long>(d) * dv + w + d;
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
  // every array starts on a 16-byte boundary where d is a multiple of 4 (the copies in 16 bytes need no
  // more: the decayed sum's d * dv array is read with plain loads)
  p.Ke = s; s += ch * pmm::kChunk * d;
  p.Qg = s; s += ch * pmm::kChunk * d;
  p.B = s; s += ch * pmm::kChunk * pmm::kChunk;
  p.N = s; s += ch * static_cast<size_t>(d) * dv;
  if (delta) {
    p.W = s; s += ch * pmm::kChunk * d;
    p.M = s; s += ch * static_cast<size_t>(d) * d;
  }
  p.Uv = s; s += ch * pmm::kChunk * dv;
  p.Eg = s;
  p.state = state; p.slots = slots; p.out = out;
  PMM_DISPATCH_DTYPE(dtype, S, {
    return delta ? pmm::launch_chunked<S, true>(p, n_chunks, stream) : pmm::launch_chunked<S, false>(p, n_chunks, stream);
  });
  return 0;
}
