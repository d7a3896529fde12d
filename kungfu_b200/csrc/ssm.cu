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
// Work split: a block of 128 threads owns (request, head, 32 values of p).  Thread (pl, ns) keeps S[n][p] for two values
// of p and every n whose group of four, n / 4, is ns modulo 8: up to 64 numbers in registers, as pairs of neighbouring
// states that one packed instruction (fma.rn.f32x2) updates together; the eight lanes that share a pair of columns add
// their partial sums of S^T C by shuffles (odd lanes take one column, even lanes the other, after the first exchange).
// Rows are staged in shared memory, B, C, x and dt as they stand in global memory, by cp.async (16 bytes where offsets
// allow, else 4) into a ring of two stages, so that the next rows arrive while the current ones are walked; the walk reads
// 16-byte vectors (eight neighbouring lanes read 128 contiguous bytes) and issues three packed instructions per pair of
// states and no global load.  Shared rows are padded with zeros to a multiple of 32 states: padded states stay zero and
// add nothing, so the walk has no bounds checks.  (Sixteen lanes per column pair, i.e. twice the warps with half the
// states each, walk one prompt no faster and several prompts a quarter slower: the work per row that does not shrink
// with the tile, shared loads, shuffles and address arithmetic, is then paid twice.)
// State layout: state[slot][head][p][n], n fastest.
#include "common.cuh"

constexpr int SSM_PC = 32;        // values of p per block
constexpr int SSM_NS = 8;         // lanes that share a pair of p
constexpr int SSM_THREADS = (SSM_PC / 2) * SSM_NS;
constexpr int SSM_MAX_N = 256;

__device__ __forceinline__ void ssm_cp4(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ssm_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void ssm_cp16(float* dst, const float* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
template <int N> __device__ __forceinline__ void ssm_cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// K4: groups of four states per thread (the padded state size is 64 * K4); ROWS: rows per stage.
template <int K4, int ROWS, typename TW>
__global__ void __launch_bounds__(SSM_THREADS, 4)
ssm_scan_kernel(const float* __restrict__ xbc, int ld_x, const float* __restrict__ proj, int ld_p, int dt_col0,
                const TW* __restrict__ dt_bias, const TW* __restrict__ a_log, const TW* __restrict__ d_skip,
                float* __restrict__ state, float* __restrict__ y, int heads, int groups, int P, int N,
                int n_reqs, const int* __restrict__ req_row_start, const int* __restrict__ req_n_rows,
                const int* __restrict__ req_state_slot, int write_state, int vec) {
  constexpr int NP = 4 * SSM_NS * K4;                         // padded state size
  constexpr int ROW_F = 2 * NP + SSM_PC + 4;                  // floats of one staged row: B | C | x | dt, decay, -, -
  kf_pdl_wait();
  __shared__ __align__(16) float stage[2][ROWS][ROW_F];
  const int req = blockIdx.x / heads, h = blockIdx.x - req * heads;
  if (req >= n_reqs) return;
  const int n_rows = req_n_rows[req];
  if (n_rows <= 0) return;                                   // a request slot of a padded layout
  const int row0 = req_row_start[req], slot = req_state_slot[req];
  const int g = h / (heads / groups);
  const int inner = heads * P;
  const int tid = threadIdx.x, ns = tid & (SSM_NS - 1), pl = tid / SSM_NS;
  const int pbase = blockIdx.y * SSM_PC;
  const int p0 = pbase + 2 * pl;

  // the zero padding: states N..NP-1 of B and C, and x beyond P (copies never write there)
  const int pad_n = NP - N, px = min(SSM_PC, P - pbase), pad_x = SSM_PC - px;
  for (int i = tid; i < 2 * ROWS * (2 * pad_n + pad_x); i += SSM_THREADS) {
    const int r = i / (2 * pad_n + pad_x), j = i - r * (2 * pad_n + pad_x);
    float* dst = (&stage[0][0][0]) + (size_t)r * ROW_F;
    if (j < pad_n) dst[N + j] = 0.f;
    else if (j < 2 * pad_n) dst[NP + N + j - pad_n] = 0.f;
    else dst[2 * NP + px + j - 2 * pad_n] = 0.f;
  }
  float2 S0[2 * K4], S1[2 * K4];                               // pairs of neighbouring states, for p0 and p0 + 1
  float* sp0 = state + (((size_t)slot * heads + h) * P + p0) * N;
#pragma unroll
  for (int k = 0; k < K4; ++k)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = 4 * (ns + SSM_NS * k) + j;
      const float v0 = (p0 < P && n < N) ? sp0[n] : 0.f, v1 = (p0 + 1 < P && n < N) ? sp0[N + n] : 0.f;
      if (j & 1) { S0[2 * k + (j >> 1)].y = v0; S1[2 * k + (j >> 1)].y = v1; }
      else { S0[2 * k + (j >> 1)].x = v0; S1[2 * k + (j >> 1)].x = v1; }
    }
  const float a = -expf(kf_load(a_log, h)), bias = kf_load(dt_bias, h), dsk = kf_load(d_skip, h);
  __syncthreads();

  const int nq = N >> 2, xq = px >> 2, items = 2 * nq + xq + 1;
  auto load = [&](int s, int i0) {                            // rows i0.. of the request into stage s
    const int nr = min(ROWS, n_rows - i0);
    if (vec) {                                                // 16 bytes at a time: sizes and offsets are multiples of four floats
      for (int idx = tid; idx < nr * items; idx += SSM_THREADS) {
        const int r = idx / items, it = idx - r * items;
        const float* row = xbc + (size_t)(row0 + i0 + r) * ld_x;
        float* dst = stage[s][r];
        if (it < nq) ssm_cp16(dst + 4 * it, row + inner + g * N + 4 * it);
        else if (it < 2 * nq) ssm_cp16(dst + NP + 4 * (it - nq), row + inner + (groups + g) * N + 4 * (it - nq));
        else if (it < 2 * nq + xq) ssm_cp16(dst + 2 * NP + 4 * (it - 2 * nq), row + h * P + pbase + 4 * (it - 2 * nq));
        else ssm_cp4(dst + 2 * NP + SSM_PC, proj + (size_t)(row0 + i0 + r) * ld_p + dt_col0 + h);
      }
    } else {
      for (int r = 0; r < nr; ++r) {
        const float* row = xbc + (size_t)(row0 + i0 + r) * ld_x;
        float* dst = stage[s][r];
        for (int n = tid; n < N; n += SSM_THREADS) {
          ssm_cp4(dst + n, row + inner + g * N + n);
          ssm_cp4(dst + NP + n, row + inner + (groups + g) * N + n);
        }
        if (tid < SSM_PC && pbase + tid < P) ssm_cp4(dst + 2 * NP + tid, row + h * P + pbase + tid);
        if (tid == SSM_PC) ssm_cp4(dst + 2 * NP + SSM_PC, proj + (size_t)(row0 + i0 + r) * ld_p + dt_col0 + h);
      }
    }
    ssm_cp_commit();
  };

  load(0, 0);
  int s = 0;
  float* yo = y + (size_t)row0 * inner + h * P + p0 + (ns & 1);          // where lane ns < 2 stores column p0 + ns
  for (int i0 = 0; i0 < n_rows; i0 += ROWS, s ^= 1) {
    const int nr = min(ROWS, n_rows - i0);
    const bool more = i0 + ROWS < n_rows;
    if (more) load(s ^ 1, i0 + ROWS);                         // that stage was walked two rounds ago (barrier at the loop's end)
    if (more) ssm_cp_wait<1>(); else ssm_cp_wait<0>();
    __syncthreads();
    if (tid < nr) {
      float* t = stage[s][tid] + 2 * NP + SSM_PC;
      const float z = t[0] + bias;
      const float dt = z > 20.f ? z + log1pf(expf(-z)) : log1pf(expf(z));
      t[0] = dt;
      t[1] = expf(a * dt);
    }
    __syncthreads();
#pragma unroll 4
    for (int r = 0; r < nr; ++r) {
      const float* row = stage[s][r];
      const float dt = row[2 * NP + SSM_PC], da = row[2 * NP + SSM_PC + 1];
      const float2 xv = *reinterpret_cast<const float2*>(row + 2 * NP + 2 * pl);
      const float2 u0 = make_float2(dt * xv.x, dt * xv.x), u1 = make_float2(dt * xv.y, dt * xv.y), dd = make_float2(da, da);
      float2 a0 = make_float2(0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll
      for (int k = 0; k < K4; ++k) {                          // two states per instruction (fma.rn.f32x2)
        const float4 b = *reinterpret_cast<const float4*>(row + 4 * (ns + SSM_NS * k));
        const float4 c = *reinterpret_cast<const float4*>(row + NP + 4 * (ns + SSM_NS * k));
        const float2 blo = make_float2(b.x, b.y), bhi = make_float2(b.z, b.w), clo = make_float2(c.x, c.y), chi = make_float2(c.z, c.w);
        S0[2 * k] = __ffma2_rn(S0[2 * k], dd, __fmul2_rn(blo, u0));          a0 = __ffma2_rn(S0[2 * k], clo, a0);
        S1[2 * k] = __ffma2_rn(S1[2 * k], dd, __fmul2_rn(blo, u1));          a1 = __ffma2_rn(S1[2 * k], clo, a1);
        S0[2 * k + 1] = __ffma2_rn(S0[2 * k + 1], dd, __fmul2_rn(bhi, u0));  a2 = __ffma2_rn(S0[2 * k + 1], chi, a2);
        S1[2 * k + 1] = __ffma2_rn(S1[2 * k + 1], dd, __fmul2_rn(bhi, u1));  a3 = __ffma2_rn(S1[2 * k + 1], chi, a3);
      }
      const float acc0 = (a0.x + a0.y) + (a2.x + a2.y), acc1 = (a1.x + a1.y) + (a3.x + a3.y);
      // the sum over the lanes of a pair of columns: odd lanes take over the second column, even lanes the first, then
      // one value per lane goes through the remaining steps
      float v = ((ns & 1) ? acc1 : acc0) + __shfl_xor_sync(0xffffffffu, (ns & 1) ? acc0 : acc1, 1);
#pragma unroll
      for (int o = 2; o < SSM_NS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (ns < 2 && p0 + ns < P) yo[(size_t)r * inner] = fmaf(dsk, ns ? xv.y : xv.x, v);
    }
    yo += (size_t)nr * inner;
    __syncthreads();                                          // everyone is done with stage s before it is loaded again
  }
  // Dependents are let in only now: this kernel runs for hundreds of microseconds with one to four blocks per SM, and a
  // dependent grid released at its start parks its blocks on every SM for all that time (measured on the 8-layer step:
  // 13.9 ms against 11.7 ms when every launch waits for the one before it).
  kf_pdl_trigger();
  if (write_state) {
#pragma unroll
    for (int k = 0; k < K4; ++k)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = 4 * (ns + SSM_NS * k) + j;
        const float2 v0 = S0[2 * k + (j >> 1)], v1 = S1[2 * k + (j >> 1)];
        if (p0 < P && n < N) sp0[n] = (j & 1) ? v0.y : v0.x;
        if (p0 + 1 < P && n < N) sp0[N + n] = (j & 1) ? v1.y : v1.x;
      }
  }
}

// One row per request (decoding): nothing is staged; every thread fetches its states, its part of B and C and the row's
// x and dt straight from global memory, all loads in flight at once.  Same split of the work and the same order of sums
// as the walk above, so a token gives the same bits whether it came alone or in a portion.
template <int K4, typename TW>
__global__ void __launch_bounds__(SSM_THREADS)
ssm_step_kernel(const float* __restrict__ xbc, int ld_x, const float* __restrict__ proj, int ld_p, int dt_col0,
                const TW* __restrict__ dt_bias, const TW* __restrict__ a_log, const TW* __restrict__ d_skip,
                float* __restrict__ state, float* __restrict__ y, int heads, int groups, int P, int N,
                int n_reqs, const int* __restrict__ req_row_start, const int* __restrict__ req_n_rows,
                const int* __restrict__ req_state_slot, int write_state) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int req = blockIdx.x / heads, h = blockIdx.x - req * heads;
  if (req >= n_reqs || req_n_rows[req] <= 0) return;
  const int t = req_row_start[req], slot = req_state_slot[req];
  const int g = h / (heads / groups);
  const int inner = heads * P;
  const int tid = threadIdx.x, ns = tid & (SSM_NS - 1), pl = tid / SSM_NS;
  const int p0 = blockIdx.y * SSM_PC + 2 * pl;
  const float* row = xbc + (size_t)t * ld_x;
  float* sp0 = state + (((size_t)slot * heads + h) * P + p0) * N;
  float2 S0[2 * K4], S1[2 * K4], bb[2 * K4], cc[2 * K4];
#pragma unroll
  for (int k = 0; k < K4; ++k)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = 4 * (ns + SSM_NS * k) + j;
      const bool in = n < N;
      const float v0 = (p0 < P && in) ? sp0[n] : 0.f, v1 = (p0 + 1 < P && in) ? sp0[N + n] : 0.f;
      const float b = in ? row[inner + g * N + n] : 0.f, c = in ? row[inner + (groups + g) * N + n] : 0.f;
      if (j & 1) { S0[2 * k + (j >> 1)].y = v0; S1[2 * k + (j >> 1)].y = v1; bb[2 * k + (j >> 1)].y = b; cc[2 * k + (j >> 1)].y = c; }
      else { S0[2 * k + (j >> 1)].x = v0; S1[2 * k + (j >> 1)].x = v1; bb[2 * k + (j >> 1)].x = b; cc[2 * k + (j >> 1)].x = c; }
    }
  const float x0 = p0 < P ? row[h * P + p0] : 0.f, x1 = p0 + 1 < P ? row[h * P + p0 + 1] : 0.f;
  const float z = proj[(size_t)t * ld_p + dt_col0 + h] + kf_load(dt_bias, h);
  const float dt = z > 20.f ? z + log1pf(expf(-z)) : log1pf(expf(z));
  const float da = expf(-expf(kf_load(a_log, h)) * dt);
  const float2 u0 = make_float2(dt * x0, dt * x0), u1 = make_float2(dt * x1, dt * x1), dd = make_float2(da, da);
  float2 a0 = make_float2(0.f, 0.f), a1 = a0, a2 = a0, a3 = a0;
#pragma unroll
  for (int k = 0; k < K4; ++k) {
    S0[2 * k] = __ffma2_rn(S0[2 * k], dd, __fmul2_rn(bb[2 * k], u0));              a0 = __ffma2_rn(S0[2 * k], cc[2 * k], a0);
    S1[2 * k] = __ffma2_rn(S1[2 * k], dd, __fmul2_rn(bb[2 * k], u1));              a1 = __ffma2_rn(S1[2 * k], cc[2 * k], a1);
    S0[2 * k + 1] = __ffma2_rn(S0[2 * k + 1], dd, __fmul2_rn(bb[2 * k + 1], u0));  a2 = __ffma2_rn(S0[2 * k + 1], cc[2 * k + 1], a2);
    S1[2 * k + 1] = __ffma2_rn(S1[2 * k + 1], dd, __fmul2_rn(bb[2 * k + 1], u1));  a3 = __ffma2_rn(S1[2 * k + 1], cc[2 * k + 1], a3);
  }
  const float acc0 = (a0.x + a0.y) + (a2.x + a2.y), acc1 = (a1.x + a1.y) + (a3.x + a3.y);
  float v = ((ns & 1) ? acc1 : acc0) + __shfl_xor_sync(0xffffffffu, (ns & 1) ? acc0 : acc1, 1);
#pragma unroll
  for (int o = 2; o < SSM_NS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (ns < 2 && p0 + ns < P) y[(size_t)t * inner + h * P + p0 + ns] = fmaf(kf_load(d_skip, h), ns ? x1 : x0, v);
  if (write_state) {
#pragma unroll
    for (int k = 0; k < K4; ++k)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = 4 * (ns + SSM_NS * k) + j;
        const float2 v0 = S0[2 * k + (j >> 1)], v1 = S1[2 * k + (j >> 1)];
        if (p0 < P && n < N) sp0[n] = (j & 1) ? v0.y : v0.x;
        if (p0 + 1 < P && n < N) sp0[N + n] = (j & 1) ? v1.y : v1.x;
      }
  }
}

KF_API int kf_ssm_scan(const float* xbc, int ld_x, const float* proj, int ld_p, int dt_col0, const void* dt_bias,
                       const void* a_log, const void* d_skip, int w_dtype, float* state, float* y, int heads, int groups,
                       int P, int N, int n_reqs, const int* req_row_start, const int* req_n_rows,
                       const int* req_state_slot, int write_state, int single_rows, cudaStream_t stream) {
  if (n_reqs <= 0) return KF_OK;
  if (N < 1 || N > SSM_MAX_N || P < 1 || heads < 1 || groups < 1 || heads % groups) return KF_ERR_SIZE;
  const dim3 grid(n_reqs * heads, kf_ceil_div(P, SSM_PC)), block(SSM_THREADS);
  // 16-byte copies when every offset into the rows is a multiple of four floats
  const int vec = (N % 4 == 0 && P % 4 == 0 && ld_x % 4 == 0 && ((uintptr_t)xbc & 15) == 0) ? 1 : 0;
// The staged walk is launched WITHOUT the programmatic-dependent-launch attribute: released early by its predecessor,
// its blocks (37 KB of shared memory and a quarter of an SM's registers each) would sit on every SM waiting while the
// kernels before it still need the room; measured on an 8-layer prompt step, 8.3 ms with the attribute, 6.5 ms without.
#define KF_GO2(K4, ROWS, TW)                                                                                            \
  ssm_scan_kernel<K4, ROWS, TW><<<grid, block, 0, stream>>>(xbc, ld_x, proj, ld_p, dt_col0, (const TW*)dt_bias,          \
            (const TW*)a_log, (const TW*)d_skip, state, y, heads, groups, P, N, n_reqs, req_row_start, req_n_rows,      \
            req_state_slot, write_state, vec)
#define KF_STEP(K4, TW)                                                                                                 \
  kf_launch(ssm_step_kernel<K4, TW>, grid, block, 0, stream, xbc, ld_x, proj, ld_p, dt_col0, (const TW*)dt_bias,         \
            (const TW*)a_log, (const TW*)d_skip, state, y, heads, groups, P, N, n_reqs, req_row_start, req_n_rows,      \
            req_state_slot, write_state)
#define KF_GO(TW)                                      \
  do {                                                 \
    if (single_rows) {                                 \
      if (N <= 32) KF_STEP(1, TW);                     \
      else if (N <= 64) KF_STEP(2, TW);                \
      else if (N <= 128) KF_STEP(4, TW);               \
      else KF_STEP(8, TW);                             \
    } else                                             \
    if (N <= 32) KF_GO2(1, 16, TW);                    \
    else if (N <= 64) KF_GO2(2, 16, TW);               \
    else if (N <= 128) KF_GO2(4, 16, TW);              \
    else KF_GO2(8, 8, TW);                             \
  } while (0)
  if (w_dtype == KF_F32) KF_GO(float);
  else if (w_dtype == KF_BF16) KF_GO(__nv_bfloat16);
  else return KF_ERR_DTYPE;
#undef KF_GO
#undef KF_GO2
#undef KF_STEP
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
