// Residual streams kept in several lanes (hyper-connections), and the sum of normed branches.
//
// hc_mix_norm: a layer's residual state is n lanes x_0..x_{n-1} of [T, D] floats.  A sublayer
// reads u = sum_s in[s] x_s through an RMS norm and its result y comes back into every lane:
//   x_t <- sum_s mix[s, t] x_s + out[t] y      (all lanes at once from the old ones)
// One launch folds the result of the sublayer before (optional) into the lanes and writes the
// normed input of the next sublayer (optional), so the lanes are read and written once per
// sublayer, as the single-stream norm kernel does with its pending branches.  With a row list
// the lanes are left alone and only the listed rows are normed (the model's last norm).
// Everything is float arithmetic; y and the normed rows have the storage type.
//
// normed_sum: out = scale * sum_b rmsnorm(x_b + bias_b) * w_b for up to four branches of one width.
#include "common.cuh"

namespace pmm {

constexpr int kMaxLanes = 8;
constexpr int kMaxBranches = 4;

// NL: an upper bound of the lane count that sizes the registers (2, 4 or 8)
template <typename S, typename Y, bool VEC, int NL>
__global__ void __launch_bounds__(256)
    hc_mix_norm_kernel(const float* x_in, long long in_lane_stride, float* x_out,
                       long long out_lane_stride, int n_lanes, const Y* __restrict__ y,
                       const float* __restrict__ mix, const float* __restrict__ out_w,
                       const float* __restrict__ in_w, const float* __restrict__ norm_w, float eps,
                       S* __restrict__ normed, const int* __restrict__ rows, int D) {
  extern __shared__ float u_row[];
  __shared__ float red[32];
  __shared__ float s_mix[kMaxLanes * kMaxLanes], s_out[kMaxLanes], s_in[kMaxLanes];
  pdl_launch_dependents();
  if (threadIdx.x < n_lanes * n_lanes) s_mix[threadIdx.x] = y ? mix[threadIdx.x] : 0.f;
  if (threadIdx.x < n_lanes) {
    s_out[threadIdx.x] = y ? out_w[threadIdx.x] : 0.f;
    s_in[threadIdx.x] = in_w ? in_w[threadIdx.x] : 0.f;
  }
  pdl_wait();
  __syncthreads();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;
  float ss = 0.f;
  const bool write_lanes = x_out && !rows && (y || x_out != x_in || in_lane_stride != out_lane_stride);
  // one element of every lane at a time; four neighbouring ones (16-byte accesses) where VEC is set
  auto element = [&](int d, const float* xo, float yv, float* xn) {
    if (y) {
#pragma unroll
      for (int to = 0; to < NL; ++to) {
        if (to < n_lanes) {
          float a = 0.f;
#pragma unroll
          for (int s = 0; s < NL; ++s)
            if (s < n_lanes) a += s_mix[s * n_lanes + to] * xo[s];
          xn[to] = a + s_out[to] * yv;
        }
      }
    } else {
#pragma unroll
      for (int s = 0; s < NL; ++s)
        if (s < n_lanes) xn[s] = xo[s];
    }
    if (normed) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < NL; ++s)
        if (s < n_lanes) u += s_in[s] * xn[s];
      u_row[d] = u;
      ss += u * u;
    }
  };
  if (VEC) {
    for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
      float xo[4][NL], xn[4][NL], yv[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int s = 0; s < NL; ++s) {
        if (s < n_lanes) {
          const float4 v = *reinterpret_cast<const float4*>(x_in + s * in_lane_stride + static_cast<long long>(t) * D + d);
          xo[0][s] = v.x; xo[1][s] = v.y; xo[2][s] = v.z; xo[3][s] = v.w;
        }
      }
      if (y) {
#pragma unroll
        for (int e = 0; e < 4; ++e) yv[e] = ldf(y + static_cast<size_t>(t) * D + d + e);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) element(d + e, xo[e], yv[e], xn[e]);
      if (write_lanes) {
#pragma unroll
        for (int s = 0; s < NL; ++s)
          if (s < n_lanes)
            *reinterpret_cast<float4*>(x_out + s * out_lane_stride + static_cast<long long>(t) * D + d) =
                make_float4(xn[0][s], xn[1][s], xn[2][s], xn[3][s]);
      }
    }
  } else {
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      float xo[NL], xn[NL];
#pragma unroll
      for (int s = 0; s < NL; ++s)
        if (s < n_lanes) xo[s] = x_in[s * in_lane_stride + static_cast<long long>(t) * D + d];
      element(d, xo, y ? ldf(y + static_cast<size_t>(t) * D + d) : 0.f, xn);
      if (write_lanes) {
#pragma unroll
        for (int s = 0; s < NL; ++s)
          if (s < n_lanes) x_out[s * out_lane_stride + static_cast<long long>(t) * D + d] = xn[s];
      }
    }
  }
  if (!normed) return;
  const float total = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(D) + eps);
  for (int d = threadIdx.x; d < D; d += blockDim.x)
    stf(normed + static_cast<size_t>(r) * D + d, u_row[d] * inv * norm_w[d]);
}

struct Branches {
  const void* x[kMaxBranches];
  long long ld[kMaxBranches];
  const float* w[kMaxBranches];
  const float* bias[kMaxBranches];  // added to the branch before its norm, or nullptr
};

template <typename S, typename O>
__global__ void __launch_bounds__(256)
    normed_sum_kernel(Branches b, int n, float eps, float scale, O* __restrict__ out, int D) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  float inv[kMaxBranches];
#pragma unroll
  for (int i = 0; i < kMaxBranches; ++i) {
    if (i < n) {
      const S* x = static_cast<const S*>(b.x[i]) + static_cast<long long>(t) * b.ld[i];
      float ss = 0.f;
      for (int d = threadIdx.x; d < D; d += blockDim.x) {
        const float v = ldf(x + d) + (b.bias[i] ? b.bias[i][d] : 0.f);
        ss += v * v;
      }
      inv[i] = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(D) + eps);
    }
  }
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float a = 0.f;
#pragma unroll
    for (int i = 0; i < kMaxBranches; ++i)
      if (i < n)
        a += (ldf(static_cast<const S*>(b.x[i]) + static_cast<long long>(t) * b.ld[i] + d) + (b.bias[i] ? b.bias[i][d] : 0.f)) *
             inv[i] * b.w[i][d];
    stf(out + static_cast<size_t>(t) * D + d, a * scale);
  }
}

}  // namespace pmm

// x_in: lane s at x_in + s*in_lane_stride (stride 0: every lane reads the same [T, D]); x_out likewise
// (nullptr: lanes are not written).  y (nullptr: nothing to fold in), mix [n, n] as [from, to], out_w [n].
// y has the type y_dtype, the normed rows the type dtype.  in_w [n], norm_w [D], normed [R, D] (nullptr: no norm).  rows: R row indices, or nullptr for all T rows.
PMM_EXPORT int pmm_hc_mix_norm(const float* x_in, long long in_lane_stride, float* x_out, long long out_lane_stride,
                               int n_lanes, const void* y, const float* mix, const float* out_w, const float* in_w,
                               const float* norm_w, float eps, void* normed, const int* rows, int R, int D,
                               int dtype, int y_dtype, cudaStream_t stream) {
  if (R <= 0) return 0;
  if (n_lanes < 1 || n_lanes > pmm::kMaxLanes || D <= 0) return PMM_ERR_BAD_ARGUMENT;
  if (y && (!mix || !out_w)) return PMM_ERR_BAD_ARGUMENT;
  if (normed && (!in_w || !norm_w)) return PMM_ERR_BAD_ARGUMENT;
  const size_t smem = normed ? static_cast<size_t>(D) * sizeof(float) : 0;
  if (smem > 200 * 1024) return PMM_ERR_BAD_ARGUMENT;
  // 16-byte accesses where every row of every lane starts on such a boundary
  const bool vec = D % 4 == 0 && reinterpret_cast<uintptr_t>(x_in) % 16 == 0 && in_lane_stride % 4 == 0 &&
                   (!x_out || (reinterpret_cast<uintptr_t>(x_out) % 16 == 0 && out_lane_stride % 4 == 0));
  PMM_DISPATCH_DTYPE(dtype, S, PMM_DISPATCH_DTYPE(y_dtype, Y, {
    auto kern = vec ? (n_lanes <= 2 ? pmm::hc_mix_norm_kernel<S, Y, true, 2>
                                    : n_lanes <= 4 ? pmm::hc_mix_norm_kernel<S, Y, true, 4> : pmm::hc_mix_norm_kernel<S, Y, true, 8>)
                    : (n_lanes <= 2 ? pmm::hc_mix_norm_kernel<S, Y, false, 2>
                                    : n_lanes <= 4 ? pmm::hc_mix_norm_kernel<S, Y, false, 4> : pmm::hc_mix_norm_kernel<S, Y, false, 8>);
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      if (e != cudaSuccess) return static_cast<int>(e);
    }
    pmm::launch_pdl(kern, dim3(R), dim3(256), smem, stream, x_in, in_lane_stride, x_out, out_lane_stride, n_lanes,
                    static_cast<const Y*>(y), mix, out_w, in_w, norm_w, eps, static_cast<S*>(normed), rows, D);
  }));
  return pmm::launch_status();
}

// x[i]: [T, D] rows of stride ld[i] in the storage type; w[i]: [D] floats; bias: nullptr, or per branch [D]
// floats (or nullptr) added to the branch before its norm; out [T, D] contiguous, float when
// out_f32 is set, else the storage type.
PMM_EXPORT int pmm_normed_sum(const void* const* x, const long long* ld, const float* const* w,
                              const float* const* bias, int n, float eps,
                              float scale, void* out, int out_f32, int T, int D, int dtype, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (n < 1 || n > pmm::kMaxBranches || D <= 0) return PMM_ERR_BAD_ARGUMENT;
  pmm::Branches b{};
  for (int i = 0; i < n; ++i) {
    b.x[i] = x[i];
    b.ld[i] = ld[i];
    b.w[i] = w[i];
    b.bias[i] = bias ? bias[i] : nullptr;
  }
  PMM_DISPATCH_DTYPE(dtype, S, {
    if (out_f32)
      pmm::launch_pdl(pmm::normed_sum_kernel<S, float>, dim3(T), dim3(256), 0, stream, b, n, eps, scale,
                      static_cast<float*>(out), D);
    else
      pmm::launch_pdl(pmm::normed_sum_kernel<S, S>, dim3(T), dim3(256), 0, stream, b, n, eps, scale,
                      static_cast<S*>(out), D);
  });
  return pmm::launch_status();
}
