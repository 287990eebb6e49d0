// The statistic-free norm  y = tanh(alpha * x) * w + b  (a scalar alpha, vectors w and b), fused with
// the residual additions the way add_rmsnorm is: branch outputs wait in the storage type and are
// folded into the float stream by the launch that norms the next sublayer's input.
//
//   s   = sa * a + sb * b                       (branches; either may be absent)
//   s   = tanh(pa * s) * pw + pb                (only when a post norm is given: a sublayer's result
//                                                is normed once more before it joins the stream)
//   v   = h + s                                 (h absent: v = s)
//   h   = v                                     (rows == nullptr and there was something to add)
//   out = tanh(alpha * v) * w + bias            (when out is given)
//
// rows != nullptr: h is left untouched and out[r] comes from row rows[r].  All arithmetic is float;
// there is no reduction, so a row is spread over blockIdx.y as well where it is wide.
#include "common.cuh"

namespace pmm {

template <typename S>
__global__ void __launch_bounds__(256)
    add_tanh_norm_kernel(float* __restrict__ h, const S* __restrict__ a, float sa, const S* __restrict__ b, float sb,
                         const float* __restrict__ post_alpha, const float* __restrict__ post_w,
                         const float* __restrict__ post_b, const float* __restrict__ alpha,
                         const float* __restrict__ w, const float* __restrict__ bias, S* __restrict__ out,
                         const int* __restrict__ rows, int D) {
  pdl_launch_dependents();
  const float al = alpha ? alpha[0] : 0.f;      // constants of the model: read before the wait
  const float pal = post_alpha ? post_alpha[0] : 0.f;
  pdl_wait();
  const int r = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[r] : r) * D;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < D; i += gridDim.y * blockDim.x) {
    float s = 0.f;
    if (a) s = sa * ldf(a + src + i);
    if (b) s = s + sb * ldf(b + src + i);
    if (post_alpha) s = tanhf(pal * s) * post_w[i] + post_b[i];
    float v = h ? h[src + i] : 0.f;
    if (a || b) {
      v = v + s;
      if (h && !rows) h[src + i] = v;
    }
    if (out) stf(out + static_cast<size_t>(r) * D + i, tanhf(al * v) * w[i] + bias[i]);
  }
}

}  // namespace pmm

// h [T, D] float or nullptr; a, b [T, D] storage type or nullptr; post_* and alpha/w/bias float (alpha and
// post_alpha point to one value each); out [R, D] storage type or nullptr; rows [R] or nullptr (then R = T).
PMM_EXPORT int pmm_add_tanh_norm(void* h, const void* a, float sa, const void* b, float sb, const float* post_alpha,
                                 const float* post_w, const float* post_b, const float* alpha, const float* w,
                                 const float* bias, void* out, const int* rows, int R, int D, int dtype,
                                 cudaStream_t stream) {
  if (R <= 0) return 0;
  if (D <= 0 || (out && !(alpha && w && bias)) || (post_alpha && !(post_w && post_b)) || (rows && !out))
    return PMM_ERR_BAD_ARGUMENT;
  int ytiles = (D + 1023) / 1024;
  if (ytiles > 64) ytiles = 64;
  PMM_DISPATCH_DTYPE(dtype, S, pmm::launch_pdl(pmm::add_tanh_norm_kernel<S>, dim3(R, ytiles), dim3(256), 0, stream,
                                               static_cast<float*>(h), static_cast<const S*>(a), sa,
                                               static_cast<const S*>(b), sb, post_alpha, post_w, post_b, alpha, w, bias,
                                               static_cast<S*>(out), rows, D));
  return pmm::launch_status();
}
