// The norm that follows a sublayer in blocks with a norm on both sides of each sublayer:
// x += d / sqrt(mean(d^2) + eps) * w, with d the sublayer's output (float32) and x the float32
// stream. One block per row; the sum of squares is formed in an order that depends on the width
// only, and the residual sum is float32 in both precisions. Where the next sublayer's norm follows at
// once (the feed-forward's after the mixer's), the same block forms it from the row it has just
// summed: xn = x / sqrt(mean(x^2) + eps') * w', one kernel instead of two.
#include "bw_act.cuh"

namespace {

constexpr int kThreads = 256;

__global__ void __launch_bounds__(kThreads)
rmsnorm_residual_kernel(const float* __restrict__ d, const float* __restrict__ w, float* x, int width, float eps,
                        const float* __restrict__ w_next, float eps_next, act_t* xn) {
  bw::pdl_enter();
  extern __shared__ float row[];
  __shared__ float red[32];
  const size_t base = static_cast<size_t>(blockIdx.x) * width;
  float ss = 0.0f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float v = d[base + i];
    row[i] = v;
    ss = __fmaf_rn(v, v, ss);
  }
  const float inv = bw::rms_scale(bw::block_sum(ss, red), width, eps);
  float ss2 = 0.0f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float v = __fadd_rn(x[base + i], bw::rms_apply(row[i], inv, w[i]));
    x[base + i] = v;
    row[i] = v;  // (each thread reads back only what it wrote)
    ss2 = __fmaf_rn(v, v, ss2);
  }
  if (!xn) return;
  const float inv2 = bw::rms_scale(bw::block_sum(ss2, red), width, eps_next);
  for (int i = threadIdx.x; i < width; i += kThreads)
    xn[base + i] = bw::from_f<act_t>(bw::rms_apply(row[i], inv2, w_next[i]));
}

}  // namespace

// w_next, xn: the norm of the summed row into xn (activation type) as well; both null for none.
BW_API int BW_FN(rmsnorm_residual)(const float* d, const float* w, float* x, int n, int width, float eps,
                                   const float* w_next, float eps_next, void* xn, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (width <= 0 || width > 48 * 1024 / 4) {
    bw::set_error("rmsnorm_residual: width %d (1 .. 12288)", width);
    return -1;
  }
  bw::launch_pdl(rmsnorm_residual_kernel, dim3(n), dim3(kThreads), static_cast<size_t>(width) * sizeof(float), stream, d,
                 w, x, width, eps, w_next, eps_next, static_cast<act_t*>(w_next ? xn : nullptr));
  return bw::launch_status();
}
