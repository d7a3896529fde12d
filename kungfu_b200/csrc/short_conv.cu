// Short causal convolution of a step's rows (see short_conv.cuh for the rule and the state), and the kernel that
// moves the state on after the step.
//
// kf_short_conv:        out[t][c] = act(conv(t, c) + out_bias[c]) for every row t of the step; rows of one request read
//                       the rows before them in the same step, or the state.
// kf_short_conv_commit: the state of every request of the step becomes its last taps-1 inputs, one thread per
//                       (request, channel).  It runs after every reader of the old state (stream order).
// Both skip padding (rows of request -1, requests without rows).
#include "short_conv.cuh"

enum { KF_CONV_ACT_NONE = 0, KF_CONV_ACT_SILU = 1 };

// VEC channels per thread (4 when every offset is a multiple of four floats: 16-byte loads and stores), `rows_per_block`
// rows per block, so that the filter taps are fetched once and a row's look-ups (its request, where that starts, its
// slot) are spread over more work.  `commit_state` (steps in which no request has more than one row, i.e. decoding): the
// thread that has just read a channel's tail also moves it on, which saves the commit kernel; with several rows per
// request other threads may still need the old tail, so the commit stays a kernel of its own there.
template <typename TW, int VEC>
__global__ void short_conv_kernel(KfConvIn p, const TW* __restrict__ w, const TW* __restrict__ out_bias, int act,
                                  float* __restrict__ out, int ld_out, const int* __restrict__ row_req,
                                  const int* __restrict__ req_row_start, const int* __restrict__ req_state_slot, int T,
                                  int rows_per_block, float* __restrict__ commit_state) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int c0 = (blockIdx.y * blockDim.x + threadIdx.x) * VEC;
  if (c0 >= p.C) return;
  float wv[VEC][KF_MAX_TAPS], bi[VEC], bo[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) {
#pragma unroll
    for (int j = 0; j < KF_MAX_TAPS; ++j) wv[v][j] = j < p.taps ? kf_load(w, (size_t)(c0 + v) * p.taps + j) : 0.f;
    bi[v] = p.in_bias ? kf_load((const TW*)p.in_bias, c0 + v) : 0.f;
    bo[v] = out_bias ? kf_load(out_bias, c0 + v) : 0.f;
  }
  const int t_end = min(T, (int)(blockIdx.x + 1) * rows_per_block);
  for (int t = blockIdx.x * rows_per_block; t < t_end; ++t) {
    const int req = row_req[t];
    if (req < 0) continue;
    const int row0 = req_row_start[req], slot = req_state_slot[req], i = t - row0;
    float acc[VEC], u[VEC];
#pragma unroll
    for (int v = 0; v < VEC; ++v) acc[v] = 0.f;
#pragma unroll
    for (int j = 0; j < KF_MAX_TAPS; ++j) {
      if (j < p.taps) {
        const int idx = i - (p.taps - 1 - j);
        if (idx >= 0) {
          const float* src = p.in + (size_t)(row0 + idx) * p.ld + p.col0 + c0;
          if (VEC == 4) { const float4 q = *reinterpret_cast<const float4*>(src); u[0] = q.x; u[1] = q.y; u[2] = q.z; u[VEC - 1] = q.w; }
          else u[0] = src[0];
#pragma unroll
          for (int v = 0; v < VEC; ++v) u[v] += bi[v];
        } else {
          const float* src = p.state + ((size_t)slot * (p.taps - 1) + (p.taps - 1 + idx)) * p.C + c0;
          if (VEC == 4) { const float4 q = *reinterpret_cast<const float4*>(src); u[0] = q.x; u[1] = q.y; u[2] = q.z; u[VEC - 1] = q.w; }
          else u[0] = src[0];
        }
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = fmaf(wv[v][j], u[v], acc[v]);
        if (commit_state && j >= 1) {                       // one row per request: input j becomes tail entry j - 1
          float* dst = commit_state + ((size_t)slot * (p.taps - 1) + (j - 1)) * p.C + c0;
          if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(u[0], u[1], u[2], u[VEC - 1]);
          else dst[0] = u[0];
        }
      }
    }
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      acc[v] += bo[v];
      if (act == KF_CONV_ACT_SILU) acc[v] = acc[v] / (1.f + expf(-acc[v]));
    }
    float* dst = out + (size_t)t * ld_out + c0;
    if (VEC == 4) *reinterpret_cast<float4*>(dst) = make_float4(acc[0], acc[1], acc[2], acc[VEC - 1]);
    else dst[0] = acc[0];
  }
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

// commit_inline: the step has no request with more than one row; the state is then moved on here and
// kf_short_conv_commit must not run for this step.
KF_API int kf_short_conv(const float* in, int ld, int col0, const void* in_bias, const void* w, const void* out_bias,
                         int w_dtype, int C, int taps, int act, float* state, float* out, int ld_out,
                         const int* row_req, const int* req_row_start, const int* req_state_slot, int T, int commit_inline,
                         cudaStream_t stream) {
  if (T <= 0 || C <= 0) return KF_OK;
  if (taps < 1 || taps > KF_MAX_TAPS) return KF_ERR_SIZE;
  KfConvIn p{in, ld, col0, in_bias, state, C, taps};
  const bool vec = C % 4 == 0 && ld % 4 == 0 && col0 % 4 == 0 && ld_out % 4 == 0 &&
                   (((uintptr_t)in | (uintptr_t)out | (uintptr_t)state) & 15) == 0;
  const int per_thread = vec ? 4 : 1;
  const int threads = C / per_thread >= 256 ? 256 : 128;
  const int rows = T >= 1024 ? 8 : (T >= 64 ? 4 : 1);
  const dim3 grid(kf_ceil_div(T, rows), kf_ceil_div(C, threads * per_thread));
  float* commit = (commit_inline && taps > 1) ? state : nullptr;
#define KF_GO(TW, VEC)                                                                                                  \
  kf_launch(short_conv_kernel<TW, VEC>, grid, dim3(threads), 0, stream, p, (const TW*)w, (const TW*)out_bias, act, out, \
            ld_out, row_req, req_row_start, req_state_slot, T, rows, commit)
  if (w_dtype == KF_F32) { if (vec) KF_GO(float, 4); else KF_GO(float, 1); }
  else if (w_dtype == KF_BF16) { if (vec) KF_GO(__nv_bfloat16, 4); else KF_GO(__nv_bfloat16, 1); }
  else return KF_ERR_DTYPE;
#undef KF_GO
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
