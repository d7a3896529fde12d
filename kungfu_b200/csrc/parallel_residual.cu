// The residual update of a block whose branches run side by side on one normed input:
//   x[t] += a[t] + b[t]      (b may be absent), all in 32-bit,
// and, in the same pass, the RMS norm the next block starts with: next[t] = x[t] / sqrt(mean(x[t]^2) + eps) * g,
// g = w or 1 + w.  One block per row; a thread reads back only elements it wrote itself.
#include "common.cuh"

template <typename TW, typename TO>
__global__ void add2_rmsnorm_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ x,
                                    const TW* __restrict__ w, float eps, int plus_one, TO* __restrict__ out, int H) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const size_t base = (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    float v = a[base + i];
    if (b) v += b[base + i];
    v += x[base + i];
    x[base + i] = v;
    ss = fmaf(v, v, ss);
  }
  if (!out) return;
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)H + eps);
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float g = kf_load(w, i) + (plus_one ? 1.f : 0.f);
    kf_store(out, base + i, x[base + i] * inv * g);
  }
}

KF_API int kf_add2_rmsnorm(const float* a, const float* b, float* x, const void* w, int w_dtype, float eps, int plus_one,
                           void* out, int out_dtype, int T, int H, cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
#define KF_GO(TW, TO)                                                                                                   \
  kf_launch(add2_rmsnorm_kernel<TW, TO>, dim3(T), dim3(threads), 0, stream, a, b, x, (const TW*)w, eps, plus_one, (TO*)out, H)
  if (!out) KF_GO(float, float);
  else if (w_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else if (w_dtype == KF_F32 && out_dtype == KF_BF16) KF_GO(float, __nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// out[i] = act(in[i]): the activation of a feed-forward without a gate, 32-bit in, the activation dtype out.
template <typename TO>
__global__ void activation_kernel(const float* __restrict__ in, TO* __restrict__ out, size_t n, int act) {
  kf_pdl_trigger();
  kf_pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    kf_store(out, i, kf_act(in[i], act));
}

KF_API int kf_activation(const float* in, void* out, int out_dtype, long n, int act, cudaStream_t stream) {
  if (n <= 0) return KF_OK;
  const long b = (n + 255) / 256;
  const int blocks = (int)(b > kf_sm_count() * 16 ? kf_sm_count() * 16 : b);
  if (out_dtype == KF_F32) kf_launch(activation_kernel<float>, dim3(blocks), dim3(256), 0, stream, in, (float*)out, (size_t)n, act);
  else if (out_dtype == KF_BF16)
    kf_launch(activation_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, in, (__nv_bfloat16*)out, (size_t)n, act);
  else return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}
