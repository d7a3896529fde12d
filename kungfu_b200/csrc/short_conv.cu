// Short causal convolution of a step's rows (see short_conv.cuh for the rule and the state), and the kernel that
// moves the state on after the step.
//
// kf_short_conv:        out[t][c] = act(conv(t, c) + out_bias[c]) for every row t of the step, one thread per
//                       (row, channel); rows of one request read the rows before them in the same step, or the state.
// kf_short_conv_commit: the state of every request of the step becomes its last taps-1 inputs, one thread per
//                       (request, channel).  It runs after every reader of the old state (stream order).
// Both skip padding (rows of request -1, requests without rows).
#include "short_conv.cuh"

enum { KF_CONV_ACT_NONE = 0, KF_CONV_ACT_SILU = 1 };

template <typename TW>
__global__ void short_conv_kernel(KfConvIn p, const TW* __restrict__ w, const TW* __restrict__ out_bias, int act,
                                  float* __restrict__ out, int ld_out, const int* __restrict__ row_req,
                                  const int* __restrict__ req_row_start, const int* __restrict__ req_state_slot) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  const int req = row_req[t];
  if (req < 0 || c >= p.C) return;
  const int row0 = req_row_start[req], slot = req_state_slot[req];
  float v = kf_conv_value<TW>(p, w, row0, slot, t - row0, c);
  if (out_bias) v += kf_load(out_bias, c);
  if (act == KF_CONV_ACT_SILU) v = v / (1.f + expf(-v));
  out[(size_t)t * ld_out + c] = v;
}

template <typename TW>
__global__ void short_conv_commit_kernel(KfConvIn p, float* __restrict__ state, int n_reqs,
                                         const int* __restrict__ req_row_start, const int* __restrict__ req_n_rows,
                                         const int* __restrict__ req_state_slot) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int req = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (req >= n_reqs || c >= p.C) return;
  const int n = req_n_rows[req];
  if (n <= 0) return;
  const int row0 = req_row_start[req], slot = req_state_slot[req];
  float v[KF_MAX_TAPS - 1];
#pragma unroll
  for (int s = 0; s < KF_MAX_TAPS - 1; ++s)
    if (s < p.taps - 1) v[s] = kf_conv_input<TW>(p, row0, slot, n - (p.taps - 1) + s, c);   // old entries are read first
#pragma unroll
  for (int s = 0; s < KF_MAX_TAPS - 1; ++s)
    if (s < p.taps - 1) state[((size_t)slot * (p.taps - 1) + s) * p.C + c] = v[s];
}

KF_API int kf_short_conv(const float* in, int ld, int col0, const void* in_bias, const void* w, const void* out_bias,
                         int w_dtype, int C, int taps, int act, const float* state, float* out, int ld_out,
                         const int* row_req, const int* req_row_start, const int* req_state_slot, int T,
                         cudaStream_t stream) {
  if (T <= 0 || C <= 0) return KF_OK;
  if (taps < 1 || taps > KF_MAX_TAPS) return KF_ERR_SIZE;
  KfConvIn p{in, ld, col0, in_bias, state, C, taps};
  const int threads = C >= 256 ? 256 : 128;
  const dim3 grid(T, kf_ceil_div(C, threads));
  if (w_dtype == KF_F32)
    kf_launch(short_conv_kernel<float>, grid, dim3(threads), 0, stream, p, (const float*)w, (const float*)out_bias, act, out,
              ld_out, row_req, req_row_start, req_state_slot);
  else if (w_dtype == KF_BF16)
    kf_launch(short_conv_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, p, (const __nv_bfloat16*)w,
              (const __nv_bfloat16*)out_bias, act, out, ld_out, row_req, req_row_start, req_state_slot);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}

KF_API int kf_short_conv_commit(const float* in, int ld, int col0, const void* in_bias, int w_dtype, int C, int taps,
                                float* state, int n_reqs, const int* req_row_start, const int* req_n_rows,
                                const int* req_state_slot, cudaStream_t stream) {
  if (n_reqs <= 0 || C <= 0 || taps <= 1) return KF_OK;
  if (taps > KF_MAX_TAPS) return KF_ERR_SIZE;
  KfConvIn p{in, ld, col0, in_bias, state, C, taps};
  const int threads = C >= 256 ? 256 : 128;
  const dim3 grid(n_reqs, kf_ceil_div(C, threads));
  if (w_dtype == KF_F32)
    kf_launch(short_conv_commit_kernel<float>, grid, dim3(threads), 0, stream, p, state, n_reqs, req_row_start, req_n_rows,
              req_state_slot);
  else if (w_dtype == KF_BF16)
    kf_launch(short_conv_commit_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, p, state, n_reqs, req_row_start,
              req_n_rows, req_state_slot);
  else
    return KF_ERR_DTYPE;
  KF_CHECK_LAUNCH();
  return KF_OK;
}
