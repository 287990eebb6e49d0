// Linear-attention recurrences with a matrix state per head, token by token.
//
// Every head keeps S [d, dv] (floats, in the request's slot).  Two update rules:
//
//   decayed sum (DELTA = false):   S <- a S + k v^T;                      o = S^T q
//     with one decay a per head, q, k, v = silu of the projections;
//   gated delta rule (DELTA = true):
//     S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;             o = S^T q
//     with one decay per head and key channel g = exp(-exp(A_log_h) softplus(a + dt_bias)),
//     beta = sigmoid(b), q and k scaled to unit length per head (q also by q_scale):
//     x / sqrt(sum x^2 + unit_eps).  The read-out sees the current token's write.
//
// A block owns 32 columns of one head's state for one sequence and walks the sequence's tokens of
// the step in order; a portion of a prompt and a lone decoded token are the same to it.  Thread
// (column j, part p) keeps rows p, p+4, p+8, ... of column j in registers for the whole walk, so the
// state is read and written once per step; the four parts of a column sit in neighbouring lanes
// and add their partial sums with two shuffles.  Tokens are staged in groups: all threads load and
// prepare (unit lengths, decays, gates) the group's q, k, g, v in shared memory, then every warp
// walks the group on its own (no block barrier inside the walk).  All arithmetic is float.
#include "common.cuh"

namespace pmm {

constexpr int kRecCols = 32;    // state columns per block
constexpr int kRecParts = 4;    // threads that share a column
constexpr int kRecGroup = 16;   // tokens staged at a time
constexpr int kRecThreads = kRecCols * kRecParts;

__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + expf(-x)); }

struct RecArgs {
  const void* q; long long ld_q;    // [T, Hk*d]   (heads of q and k: Hk; head h reads h / (H / Hk))
  const void* k; long long ld_k;
  const void* v; long long ld_v;    // [T, H*dv]
  const void* beta; long long ld_beta;  // DELTA: [T, H]
  const void* a; long long ld_a;        // DELTA: [T, H*d]
  const float* dt_bias;             // DELTA: [H*d]
  const float* a_log;               // DELTA: [H]
  const float* decay;               // !DELTA: [H]
  float* state;                     // [slots, H, d, dv]
  const int* cu; const int* slots;
  float* out;                       // [T, H*dv]
  int H, Hk, d, dv;
  float unit_eps, q_scale;
};

template <typename S, int R, bool DELTA>
__global__ void __launch_bounds__(kRecThreads)
    recurrent_scan_kernel(RecArgs p) {
  extern __shared__ float sm[];
  const int d = p.d, dv = p.dv;
  float* s_q = sm;                          // [group][d]
  float* s_k = s_q + kRecGroup * d;         // [group][d]
  float* s_g = s_k + kRecGroup * d;         // DELTA: [group][d]
  float* s_v = s_g + (DELTA ? kRecGroup * d : 0);  // [group][32]
  float* s_b = s_v + kRecGroup * kRecCols;  // DELTA: [group]
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * kRecCols;
  const int t0 = p.cu[seq], n_tok = p.cu[seq + 1] - t0;
  if (n_tok <= 0) return;
  const int hk = h / (p.H / p.Hk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int part = lane & (kRecParts - 1);
  const int jl = warp * (32 / kRecParts) + (lane >> 2);
  const int j = j0 + jl;
  const bool col_ok = j < dv;
  float* st = p.state + ((static_cast<size_t>(p.slots[seq]) * p.H + h) * d) * dv;

  float s[R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = part + kRecParts * r;
    s[r] = (col_ok && i < d) ? st[static_cast<size_t>(i) * dv + j] : 0.f;
  }
  const float decay = DELTA ? 0.f : p.decay[h];
  const float a_neg = DELTA ? -expf(p.a_log[h]) : 0.f;
  const S* gq = static_cast<const S*>(p.q);
  const S* gk = static_cast<const S*>(p.k);
  const S* gv = static_cast<const S*>(p.v);
  const S* gb = static_cast<const S*>(p.beta);
  const S* ga = static_cast<const S*>(p.a);

  for (int g0 = 0; g0 < n_tok; g0 += kRecGroup) {
    const int n = min(kRecGroup, n_tok - g0);
    __syncthreads();  // the walk over the group before is over
    for (int e = tid; e < n * d; e += kRecThreads) {
      const int tt = e / d, i = e - tt * d;
      const long long t = t0 + g0 + tt;
      const float qv = ldf(gq + t * p.ld_q + hk * d + i), kv = ldf(gk + t * p.ld_k + hk * d + i);
      if (DELTA) {
        s_q[e] = qv;
        s_k[e] = kv;
        const float av = ldf(ga + t * p.ld_a + h * d + i) + p.dt_bias[h * d + i];
        s_g[e] = expf(a_neg * softplus_f(av));
      } else {
        s_q[e] = silu_f(qv);
        s_k[e] = silu_f(kv);
      }
    }
    for (int e = tid; e < n * kRecCols; e += kRecThreads) {
      const int tt = e / kRecCols, c = e - tt * kRecCols;
      float vv = 0.f;
      if (j0 + c < dv) {
        vv = ldf(gv + static_cast<long long>(t0 + g0 + tt) * p.ld_v + h * dv + j0 + c);
        if (!DELTA) vv = silu_f(vv);
      }
      s_v[e] = vv;
    }
    if (DELTA) {
      if (tid < n) s_b[tid] = sigmoid_f(ldf(gb + static_cast<long long>(t0 + g0 + tid) * p.ld_beta + h));
      __syncthreads();
      // unit length per token: a warp takes tokens warp, warp + 4, ...
      for (int tt = warp; tt < n; tt += kRecThreads / 32) {
        float sq = 0.f, sk = 0.f;
        for (int i = lane; i < d; i += 32) {
          const float a = s_q[tt * d + i], b = s_k[tt * d + i];
          sq += a * a;
          sk += b * b;
        }
        sq = warp_sum(sq);
        sk = warp_sum(sk);
        const float fq = p.q_scale / sqrtf(sq + p.unit_eps), fk = 1.f / sqrtf(sk + p.unit_eps);
        for (int i = lane; i < d; i += 32) {
          s_q[tt * d + i] *= fq;
          s_k[tt * d + i] *= fk;
        }
      }
    }
    __syncthreads();
    for (int tt = 0; tt < n; ++tt) {
      const float* qr = s_q + tt * d;
      const float* kr = s_k + tt * d;
      const float vj = s_v[tt * kRecCols + jl];
      float o = 0.f;
      if (DELTA) {
        const float* gr = s_g + tt * d;
        float dot = 0.f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int i = part + kRecParts * r;
          if (i < d) {
            s[r] *= gr[i];
            dot += kr[i] * s[r];
          }
        }
        dot += __shfl_xor_sync(0xffffffffu, dot, 1);
        dot += __shfl_xor_sync(0xffffffffu, dot, 2);
        const float u = s_b[tt] * (vj - dot);
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int i = part + kRecParts * r;
          if (i < d) {
            s[r] += kr[i] * u;
            o += qr[i] * s[r];
          }
        }
      } else {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int i = part + kRecParts * r;
          if (i < d) {
            s[r] = decay * s[r] + kr[i] * vj;
            o += qr[i] * s[r];
          }
        }
      }
      o += __shfl_xor_sync(0xffffffffu, o, 1);
      o += __shfl_xor_sync(0xffffffffu, o, 2);
      if (part == 0 && col_ok) p.out[static_cast<size_t>(t0 + g0 + tt) * (p.H * dv) + h * dv + j] = o;
    }
  }
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = part + kRecParts * r;
    if (col_ok && i < d) st[static_cast<size_t>(i) * dv + j] = s[r];
  }
}

template <typename S, bool DELTA>
int launch_recurrent(const RecArgs& a, int n_seq, cudaStream_t stream) {
  const int d = a.d;
  dim3 grid((a.dv + kRecCols - 1) / kRecCols, a.H, n_seq);
  const size_t smem = sizeof(float) * (static_cast<size_t>(kRecGroup) * d * (DELTA ? 3 : 2) +
                                       kRecGroup * kRecCols + kRecGroup);
#define PMM_REC_CASE(RR)                                                                             \
  do {                                                                                               \
    auto kern = recurrent_scan_kernel<S, RR, DELTA>;                                                 \
    if (smem > 48 * 1024) {                                                                          \
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,        \
                                           static_cast<int>(smem));                                  \
      if (e != cudaSuccess) return static_cast<int>(e);                                              \
    }                                                                                                \
    launch_pdl(kern, grid, dim3(kRecThreads), smem, stream, a);                                      \
  } while (0)
  if (d <= 32) PMM_REC_CASE(8);
  else if (d <= 64) PMM_REC_CASE(16);
  else if (d <= 128) PMM_REC_CASE(32);
  else PMM_REC_CASE(64);
#undef PMM_REC_CASE
  return launch_status();
}

}  // namespace pmm

// Key sizes d up to 256, any value size.  q, k: [T, Hk*d] rows of stride ld (storage type); v [T, H*dv];
// state [slots, H, d, dv] floats; out [T, H*dv] floats; cu [n_seq + 1], slots [n_seq].
PMM_EXPORT int pmm_delta_scan(const void* q, long long ld_q, const void* k, long long ld_k, const void* v,
                              long long ld_v, const void* beta, long long ld_beta, const void* a, long long ld_a,
                              const float* dt_bias, const float* a_log, float* state, const int* cu,
                              const int* slots, float* out, int n_seq, int H, int Hk, int d, int dv,
                              float unit_eps, float q_scale, int dtype, cudaStream_t stream) {
  if (n_seq <= 0) return 0;
  if (H <= 0 || Hk <= 0 || H % Hk || d <= 0 || d > 256 || dv <= 0 || H > 65535 || n_seq > 65535)
    return PMM_ERR_BAD_ARGUMENT;
  pmm::RecArgs p{q, ld_q, k, ld_k, v, ld_v, beta, ld_beta, a, ld_a, dt_bias, a_log, nullptr, state, cu, slots, out,
                 H, Hk, d, dv, unit_eps, q_scale};
  PMM_DISPATCH_DTYPE(dtype, S, return (pmm::launch_recurrent<S, true>(p, n_seq, stream)));
  return 0;
}

PMM_EXPORT int pmm_decay_scan(const void* q, long long ld_q, const void* k, long long ld_k, const void* v,
                              long long ld_v, const float* decay, float* state, const int* cu, const int* slots,
                              float* out, int n_seq, int H, int d, int dv, int dtype, cudaStream_t stream) {
  if (n_seq <= 0) return 0;
  if (H <= 0 || d <= 0 || d > 256 || dv <= 0 || H > 65535 || n_seq > 65535) return PMM_ERR_BAD_ARGUMENT;
  pmm::RecArgs p{q, ld_q, k, ld_k, v, ld_v, nullptr, 0, nullptr, 0, nullptr, nullptr, decay, state, cu, slots, out,
                 H, H, d, dv, 0.f, 1.f};
  PMM_DISPATCH_DTYPE(dtype, S, return (pmm::launch_recurrent<S, false>(p, n_seq, stream)));
  return 0;
}
