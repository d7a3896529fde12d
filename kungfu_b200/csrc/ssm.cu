// The recurrence of a Mamba-2 style state-space mixer, and the gated group norm that follows it.
//
// Per head h (which reads group g = h / (heads / groups) of B and C) and token t of a request, with the state S an
// N x P matrix of 32-bit floats kept per request between steps:
//   dt  = softplus(dt_raw[t][h] + dt_bias[h])                       (log1p(exp(.)), no clamp)
//   S   = exp(-exp(A_log[h]) * dt) * S + dt * B_t (x_t)^T          (B_t: N numbers of group g, x_t: P numbers of head h)
//   y_t = S^T C_t + D[h] * x_t
// x, B, C come from one 32-bit matrix (the output of the short convolution and its activation) laid out as
// [ heads*P | groups*N | groups*N ] per row; dt_raw is a column range of the projection's 32-bit result.
// The tokens of a request are walked in order, whatever the step holds of it (one token, a portion, a whole prompt),
// so the result at a token does not depend on how the sequence was cut.
//
// Work split: a block owns (request, head, 32 values of p); thread (p, ns) keeps S[n][p] for n = ns, ns + 8, ... in
// registers, eight neighbouring lanes share a p and add their partial sums of S^T C by shuffles.  Rows are staged
// eight at a time in shared memory (dt*B, C, x, the decay), so the walk itself issues no global loads.
// State layout: state[slot][head][p][n], n fastest.
#include "common.cuh"

constexpr int SSM_PC = 32;        // values of p per block
constexpr int SSM_NS = 8;         // lanes that share a p
constexpr int SSM_ROWS = 8;       // rows staged per round
constexpr int SSM_MAX_N = 256;

template <int NPER, typename TW>
__global__ void __launch_bounds__(SSM_PC * SSM_NS)
ssm_scan_kernel(const float* __restrict__ xbc, int ld_x, const float* __restrict__ proj, int ld_p, int dt_col0,
                const TW* __restrict__ dt_bias, const TW* __restrict__ a_log, const TW* __restrict__ d_skip,
                float* __restrict__ state, float* __restrict__ y, int heads, int groups, int P, int N,
                int n_reqs, const int* __restrict__ req_row_start, const int* __restrict__ req_n_rows,
                const int* __restrict__ req_state_slot, int write_state) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float s_dtb[SSM_ROWS][SSM_MAX_N];
  __shared__ float s_c[SSM_ROWS][SSM_MAX_N];
  __shared__ float s_x[SSM_ROWS][SSM_PC];
  __shared__ float s_da[SSM_ROWS], s_dt[SSM_ROWS];
  const int req = blockIdx.x / heads, h = blockIdx.x - req * heads;
  if (req >= n_reqs) return;
  const int n_rows = req_n_rows[req];
  if (n_rows <= 0) return;                                   // a request slot of a padded layout
  const int row0 = req_row_start[req], slot = req_state_slot[req];
  const int g = h / (heads / groups);
  const int inner = heads * P;
  const int tid = threadIdx.x, ns = tid & (SSM_NS - 1), pl = tid >> 3;
  const int p = blockIdx.y * SSM_PC + pl;
  const bool live = p < P;
  float* sp = state + (((size_t)slot * heads + h) * P + (live ? p : 0)) * N;
  float S[NPER];
#pragma unroll
  for (int k = 0; k < NPER; ++k) {
    const int n = ns + SSM_NS * k;
    S[k] = (live && n < N) ? sp[n] : 0.f;
  }
  const float a = -expf(kf_load(a_log, h)), bias = kf_load(dt_bias, h), dsk = kf_load(d_skip, h);

  for (int i0 = 0; i0 < n_rows; i0 += SSM_ROWS) {
    const int nr = min(SSM_ROWS, n_rows - i0);
    __syncthreads();                                         // the round before has been read
    if (tid < nr) {
      const float z = proj[(size_t)(row0 + i0 + tid) * ld_p + dt_col0 + h] + bias;
      const float dt = z > 20.f ? z + log1pf(expf(-z)) : log1pf(expf(z));
      s_dt[tid] = dt;
      s_da[tid] = expf(a * dt);
    }
    __syncthreads();
    for (int idx = tid; idx < nr * N; idx += SSM_PC * SSM_NS) {
      const int r = idx / N, n = idx - r * N;
      const float* row = xbc + (size_t)(row0 + i0 + r) * ld_x + inner + g * N + n;
      s_dtb[r][n] = s_dt[r] * row[0];
      s_c[r][n] = row[(size_t)groups * N];
    }
    for (int idx = tid; idx < nr * SSM_PC; idx += SSM_PC * SSM_NS) {
      const int r = idx / SSM_PC, q = idx - r * SSM_PC;
      const int pp = blockIdx.y * SSM_PC + q;
      s_x[r][q] = pp < P ? xbc[(size_t)(row0 + i0 + r) * ld_x + h * P + pp] : 0.f;
    }
    __syncthreads();
    for (int r = 0; r < nr; ++r) {
      const float da = s_da[r], xp = s_x[r][pl];
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < NPER; ++k) {
        const int n = ns + SSM_NS * k;
        if (n < N) {
          S[k] = fmaf(S[k], da, s_dtb[r][n] * xp);
          acc = fmaf(S[k], s_c[r][n], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (live && ns == 0) y[(size_t)(row0 + i0 + r) * inner + h * P + p] = fmaf(dsk, xp, acc);
    }
  }
  if (write_state && live) {
#pragma unroll
    for (int k = 0; k < NPER; ++k) {
      const int n = ns + SSM_NS * k;
      if (n < N) sp[n] = S[k];
    }
  }
}

KF_API int kf_ssm_scan(const float* xbc, int ld_x, const float* proj, int ld_p, int dt_col0, const void* dt_bias,
                       const void* a_log, const void* d_skip, int w_dtype, float* state, float* y, int heads, int groups,
                       int P, int N, int n_reqs, const int* req_row_start, const int* req_n_rows,
                       const int* req_state_slot, int write_state, cudaStream_t stream) {
  if (n_reqs <= 0) return KF_OK;
  if (N < 1 || N > SSM_MAX_N || P < 1 || heads < 1 || groups < 1 || heads % groups) return KF_ERR_SIZE;
  const dim3 grid(n_reqs * heads, kf_ceil_div(P, SSM_PC)), block(SSM_PC * SSM_NS);
  const int nper = kf_ceil_div(N, SSM_NS);
#define KF_GO2(NPER, TW)                                                                                              \
  kf_launch(ssm_scan_kernel<NPER, TW>, grid, block, 0, stream, xbc, ld_x, proj, ld_p, dt_col0, (const TW*)dt_bias,    \
            (const TW*)a_log, (const TW*)d_skip, state, y, heads, groups, P, N, n_reqs, req_row_start, req_n_rows,      \
            req_state_slot, write_state)
#define KF_GO(TW)                                    \
  do {                                               \
    if (nper <= 4) KF_GO2(4, TW);                    \
    else if (nper <= 8) KF_GO2(8, TW);               \
    else if (nper <= 16) KF_GO2(16, TW);             \
    else KF_GO2(32, TW);                             \
  } while (0)
  if (w_dtype == KF_F32) KF_GO(float);
  else if (w_dtype == KF_BF16) KF_GO(__nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
#undef KF_GO2
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// out[t][j] = rms_part(y[t] * silu(z[t]))[j] * w[j]: the gate is applied first, then every one of `parts` equal parts
// of the row is divided by its own root mean square (eps inside the root).  z is columns z_col0.. of a 32-bit matrix
// with ld columns.  One block per (row, part); sums in 32-bit.
template <typename TW, typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ z, int ld, int z_col0,
                                        const TW* __restrict__ w, float eps, int inner, int parts, TO* __restrict__ out,
                                        const int* __restrict__ row_req) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  const int t = blockIdx.x, part = blockIdx.y;
  const int len = inner / parts, j0 = part * len;
  if (row_req[t] < 0) {
    for (int j = threadIdx.x; j < len; j += blockDim.x) kf_store(out, (size_t)t * inner + j0 + j, 0.f);
    return;
  }
  const float* yr = y + (size_t)t * inner + j0;
  const float* zr = z + (size_t)t * ld + z_col0 + j0;
  float ss = 0.f;
  for (int j = threadIdx.x; j < len; j += blockDim.x) {
    const float zz = zr[j];
    const float v = yr[j] * (zz / (1.f + expf(-zz)));
    ss = fmaf(v, v, ss);
  }
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)len + eps);
  for (int j = threadIdx.x; j < len; j += blockDim.x) {
    const float zz = zr[j];
    const float v = yr[j] * (zz / (1.f + expf(-zz)));
    kf_store(out, (size_t)t * inner + j0 + j, v * inv * kf_load(w, j0 + j));
  }
}

KF_API int kf_gated_group_norm(const float* y, const float* z, int ld, int z_col0, const void* w, int w_dtype, float eps,
                               int inner, int parts, void* out, int out_dtype, const int* row_req, int T,
                               cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (parts < 1 || inner % parts) return KF_ERR_SIZE;
  const int len = inner / parts;
  const int threads = len >= 1024 ? 256 : 128;
  const dim3 grid(T, parts);
#define KF_GO(TW, TO)                                                                                                \
  kf_launch(gated_group_norm_kernel<TW, TO>, grid, dim3(threads), 0, stream, y, z, ld, z_col0, (const TW*)w, eps, inner, \
            parts, (TO*)out, row_req)
  if (w_dtype == KF_F32 && out_dtype == KF_F32) KF_GO(float, float);
  else if (w_dtype == KF_BF16 && out_dtype == KF_BF16) KF_GO(__nv_bfloat16, __nv_bfloat16);
  else if (w_dtype == KF_BF16 && out_dtype == KF_F32) KF_GO(__nv_bfloat16, float);
  else return KF_ERR_DTYPE;
#undef KF_GO
  KF_CHECK_LAUNCH();
  return KF_OK;
}
