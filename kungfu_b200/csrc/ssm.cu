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

// K4: groups of four states per thread (the padded state size is 32 * K4); ROWS: rows per stage.
// STATE_ONLY: the walk of a chunk of a long prompt from a zero state, which leaves only the chunk's end state and the
// product of its decays (no C, no sums, no y); see kf_ssm_scan_chunked.
// A request (or chunk) r reads its first state from state_in[slot_in[r]] and leaves its last state in
// state_out[slot_out[r]] (slot_out[r] < 0: nowhere).
template <int K4, int ROWS, typename TW, bool STATE_ONLY>
__global__ void __launch_bounds__(SSM_THREADS, 4)
ssm_scan_kernel(const float* __restrict__ xbc, int ld_x, const float* __restrict__ proj, int ld_p, int dt_col0,
                const TW* __restrict__ dt_bias, const TW* __restrict__ a_log, const TW* __restrict__ d_skip,
                const float* __restrict__ state_in, const int* __restrict__ slot_in, float* __restrict__ state_out,
                const int* __restrict__ slot_out, float* __restrict__ decay_out, float* __restrict__ y, int heads, int groups,
                int P, int N, int n_reqs, const int* __restrict__ req_row_start, const int* __restrict__ req_n_rows,
                int write_state, int vec) {
  constexpr int NP = 4 * SSM_NS * K4;                         // padded state size
  constexpr int ROW_F = 2 * NP + SSM_PC + 4;                  // floats of one staged row: B | C | x | dt, decay, -, -
  kf_pdl_wait();
  __shared__ __align__(16) float stage[2][ROWS][ROW_F];
  const int req = blockIdx.x / heads, h = blockIdx.x - req * heads;
  if (req >= n_reqs) return;
  const int n_rows = req_n_rows[req];
  if (n_rows <= 0) return;                                   // a request slot of a padded layout
  const int row0 = req_row_start[req];
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
  const float* sp0 = STATE_ONLY ? nullptr : state_in + (((size_t)slot_in[req] * heads + h) * P + p0) * N;
#pragma unroll
  for (int k = 0; k < K4; ++k)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = 4 * (ns + SSM_NS * k) + j;
      const float v0 = (!STATE_ONLY && p0 < P && n < N) ? sp0[n] : 0.f, v1 = (!STATE_ONLY && p0 + 1 < P && n < N) ? sp0[N + n] : 0.f;
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
        else if (it < 2 * nq) { if (!STATE_ONLY) ssm_cp16(dst + NP + 4 * (it - nq), row + inner + (groups + g) * N + 4 * (it - nq)); }
        else if (it < 2 * nq + xq) ssm_cp16(dst + 2 * NP + 4 * (it - 2 * nq), row + h * P + pbase + 4 * (it - 2 * nq));
        else ssm_cp4(dst + 2 * NP + SSM_PC, proj + (size_t)(row0 + i0 + r) * ld_p + dt_col0 + h);
      }
    } else {
      for (int r = 0; r < nr; ++r) {
        const float* row = xbc + (size_t)(row0 + i0 + r) * ld_x;
        float* dst = stage[s][r];
        for (int n = tid; n < N; n += SSM_THREADS) {
          ssm_cp4(dst + n, row + inner + g * N + n);
          if (!STATE_ONLY) ssm_cp4(dst + NP + n, row + inner + (groups + g) * N + n);
        }
        if (tid < SSM_PC && pbase + tid < P) ssm_cp4(dst + 2 * NP + tid, row + h * P + pbase + tid);
        if (tid == SSM_PC) ssm_cp4(dst + 2 * NP + SSM_PC, proj + (size_t)(row0 + i0 + r) * ld_p + dt_col0 + h);
      }
    }
    ssm_cp_commit();
  };

  load(0, 0);
  int s = 0;
  float log_decay = 0.f;
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
    if (STATE_ONLY && tid == 0 && blockIdx.y == 0)
      for (int r = 0; r < nr; ++r) log_decay += a * stage[s][r][2 * NP + SSM_PC];
#pragma unroll 4
    for (int r = 0; r < nr; ++r) {
      const float* row = stage[s][r];
      const float dt = row[2 * NP + SSM_PC], da = row[2 * NP + SSM_PC + 1];
      const float2 xv = *reinterpret_cast<const float2*>(row + 2 * NP + 2 * pl);
      const float2 u0 = make_float2(dt * xv.x, dt * xv.x), u1 = make_float2(dt * xv.y, dt * xv.y), dd = make_float2(da, da);
      if (STATE_ONLY) {
#pragma unroll
        for (int k = 0; k < K4; ++k) {
          const float4 b = *reinterpret_cast<const float4*>(row + 4 * (ns + SSM_NS * k));
          const float2 blo = make_float2(b.x, b.y), bhi = make_float2(b.z, b.w);
          S0[2 * k] = __ffma2_rn(S0[2 * k], dd, __fmul2_rn(blo, u0));
          S1[2 * k] = __ffma2_rn(S1[2 * k], dd, __fmul2_rn(blo, u1));
          S0[2 * k + 1] = __ffma2_rn(S0[2 * k + 1], dd, __fmul2_rn(bhi, u0));
          S1[2 * k + 1] = __ffma2_rn(S1[2 * k + 1], dd, __fmul2_rn(bhi, u1));
        }
        continue;
      }
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
  const int so = write_state ? slot_out[req] : -1;
  if (so >= 0) {
    float* dp0 = state_out + (((size_t)so * heads + h) * P + p0) * N;
#pragma unroll
    for (int k = 0; k < K4; ++k)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = 4 * (ns + SSM_NS * k) + j;
        const float2 v0 = S0[2 * k + (j >> 1)], v1 = S1[2 * k + (j >> 1)];
        if (p0 < P && n < N) dp0[n] = (j & 1) ? v0.y : v0.x;
        if (p0 + 1 < P && n < N) dp0[N + n] = (j & 1) ? v1.y : v1.x;
      }
    if (STATE_ONLY && tid == 0 && blockIdx.y == 0) decay_out[(size_t)so * heads + h] = expf(log_decay);
  }
}

// ---- a long prompt in chunks that are walked side by side -------------------------------------------------------------
// One request's state gives few blocks, and its rows depend on one another, so a lone long prompt leaves most of the GPU
// waiting.  The recurrence is linear in the state, S_t = a_t S_(t-1) + u_t, so a prompt can be cut into chunks of L rows:
//   1. every chunk but a request's last is walked from a ZERO state, which gives its own contribution E_k to the state at
//      its end and the product D_k of its decays (the walk above in its STATE_ONLY form, all chunks side by side);
//   2. the states at the chunks' starts follow one after the other, I_(k+1) = D_k I_k + E_k, from the request's stored
//      state (an elementwise kernel, sequential over a request's chunks);
//   3. every chunk is walked from its I_k exactly as an unchunked walk would pass through it, writing y, and a
//      request's last chunk leaves the request's new state.
// The arithmetic of step 3 is that of the plain walk; only the I_k are rounded differently (sums regrouped).

__global__ void ssm_chunk_table_kernel(int n_reqs, const int* __restrict__ req_row_start, const int* __restrict__ req_n_rows,
                                       const int* __restrict__ req_state_slot, int L, int max_chunks, int* __restrict__ tab) {
  kf_pdl_trigger();
  kf_pdl_wait();
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int* c_row_start = tab;                                   // per chunk: first row, rows, rows if walked in step 1,
  int* c_n_rows = tab + max_chunks;                         // its own index, the slot its end state goes to (or -1)
  int* c_n_rows_a = tab + 2 * max_chunks;
  int* c_ident = tab + 3 * max_chunks;
  int* c_out_slot = tab + 4 * max_chunks;
  int* r_chunk0 = tab + 5 * max_chunks;                     // per request: its first chunk and how many it has
  int* r_nchunks = r_chunk0 + n_reqs;
  int k = 0;
  for (int r = 0; r < n_reqs; ++r) {
    const int n = req_n_rows[r], nc = n > 0 ? (n + L - 1) / L : 0;
    r_chunk0[r] = k;
    r_nchunks[r] = nc;
    for (int c = 0; c < nc && k < max_chunks; ++c, ++k) {
      const int rows = min(L, n - c * L);
      c_row_start[k] = req_row_start[r] + c * L;
      c_n_rows[k] = rows;
      c_n_rows_a[k] = c == nc - 1 ? 0 : rows;
      c_ident[k] = k;
      c_out_slot[k] = c == nc - 1 ? req_state_slot[r] : -1;
    }
  }
  for (; k < max_chunks; ++k) { c_row_start[k] = 0; c_n_rows[k] = 0; c_n_rows_a[k] = 0; c_ident[k] = k; c_out_slot[k] = -1; }
}

__global__ void ssm_chunk_fold_kernel(const float* __restrict__ state, float* __restrict__ chunk_state,
                                      const float* __restrict__ chunk_decay, int heads, int PN, int n_reqs,
                                      const int* __restrict__ req_state_slot, const int* __restrict__ r_chunk0,
                                      const int* __restrict__ r_nchunks) {
  kf_pdl_trigger();
  kf_pdl_wait();
  const int req = blockIdx.x, h = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  if (e >= PN) return;
  const int nc = r_nchunks[req];
  if (nc <= 0) return;
  const int k0 = r_chunk0[req];
  float S = state[((size_t)req_state_slot[req] * heads + h) * PN + e];
  for (int c = 0; c < nc; ++c) {
    float* at = chunk_state + ((size_t)(k0 + c) * heads + h) * PN + e;
    const float own = c < nc - 1 ? *at : 0.f;               // E_k, left there by step 1
    *at = S;                                                // I_k, read by step 3
    if (c < nc - 1) S = fmaf(chunk_decay[(size_t)(k0 + c) * heads + h], S, own);
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
                const int* __restrict__ req_state_slot, int write_state, int vec) {
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
  if (vec) {                                                // groups of four states in 16-byte loads (N a multiple of four)
    const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      const int n = 4 * (ns + SSM_NS * k);
      const bool in = n < N;
      const float4 v0 = (in && p0 < P) ? *reinterpret_cast<const float4*>(sp0 + n) : zero4;
      const float4 v1 = (in && p0 + 1 < P) ? *reinterpret_cast<const float4*>(sp0 + N + n) : zero4;
      const float4 b = in ? *reinterpret_cast<const float4*>(row + inner + g * N + n) : zero4;
      const float4 c = in ? *reinterpret_cast<const float4*>(row + inner + (groups + g) * N + n) : zero4;
      S0[2 * k] = make_float2(v0.x, v0.y); S0[2 * k + 1] = make_float2(v0.z, v0.w);
      S1[2 * k] = make_float2(v1.x, v1.y); S1[2 * k + 1] = make_float2(v1.z, v1.w);
      bb[2 * k] = make_float2(b.x, b.y); bb[2 * k + 1] = make_float2(b.z, b.w);
      cc[2 * k] = make_float2(c.x, c.y); cc[2 * k + 1] = make_float2(c.z, c.w);
    }
  } else
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
  if (write_state && vec) {
#pragma unroll
    for (int k = 0; k < K4; ++k) {
      const int n = 4 * (ns + SSM_NS * k);
      if (n >= N) continue;
      if (p0 < P) *reinterpret_cast<float4*>(sp0 + n) = make_float4(S0[2 * k].x, S0[2 * k].y, S0[2 * k + 1].x, S0[2 * k + 1].y);
      if (p0 + 1 < P) *reinterpret_cast<float4*>(sp0 + N + n) = make_float4(S1[2 * k].x, S1[2 * k].y, S1[2 * k + 1].x, S1[2 * k + 1].y);
    }
  } else if (write_state) {
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

// The staged walk is launched WITHOUT the programmatic-dependent-launch attribute: released early by its predecessor,
// its blocks (37 KB of shared memory and a quarter of an SM's registers each) would sit on every SM waiting while the
// kernels before it still need the room; measured on an 8-layer prompt step, 8.3 ms with the attribute, 6.5 ms without.
template <typename TW, bool STATE_ONLY>
static void ssm_launch_walk(dim3 grid, cudaStream_t stream, const float* xbc, int ld_x, const float* proj, int ld_p, int dt_col0,
                            const void* dt_bias, const void* a_log, const void* d_skip, const float* state_in, const int* slot_in,
                            float* state_out, const int* slot_out, float* decay_out, float* y, int heads, int groups, int P, int N,
                            int n_reqs, const int* row_start, const int* n_rows, int write_state, int vec) {
  const dim3 block(SSM_THREADS);
#define KF_GO2(K4, ROWS)                                                                                                 \
  ssm_scan_kernel<K4, ROWS, TW, STATE_ONLY><<<grid, block, 0, stream>>>(xbc, ld_x, proj, ld_p, dt_col0, (const TW*)dt_bias, \
      (const TW*)a_log, (const TW*)d_skip, state_in, slot_in, state_out, slot_out, decay_out, y, heads, groups, P, N, n_reqs, \
      row_start, n_rows, write_state, vec)
  if (N <= 32) KF_GO2(1, 16);
  else if (N <= 64) KF_GO2(2, 16);
  else if (N <= 128) KF_GO2(4, 16);
  else KF_GO2(8, 8);
#undef KF_GO2
}

KF_API int kf_ssm_scan(const float* xbc, int ld_x, const float* proj, int ld_p, int dt_col0, const void* dt_bias,
                       const void* a_log, const void* d_skip, int w_dtype, float* state, float* y, int heads, int groups,
                       int P, int N, int n_reqs, const int* req_row_start, const int* req_n_rows,
                       const int* req_state_slot, int write_state, int single_rows, cudaStream_t stream) {
  if (n_reqs <= 0) return KF_OK;
  if (N < 1 || N > SSM_MAX_N || P < 1 || heads < 1 || groups < 1 || heads % groups) return KF_ERR_SIZE;
  if (w_dtype != KF_F32 && w_dtype != KF_BF16) return KF_ERR_DTYPE;
  const dim3 grid(n_reqs * heads, kf_ceil_div(P, SSM_PC)), block(SSM_THREADS);
  // 16-byte copies when every offset into the rows is a multiple of four floats
  const int vec = (N % 4 == 0 && P % 4 == 0 && ld_x % 4 == 0 && ((uintptr_t)xbc & 15) == 0) ? 1 : 0;
  if (single_rows) {
#define KF_STEP(K4, TW)                                                                                                 \
  kf_launch(ssm_step_kernel<K4, TW>, grid, block, 0, stream, xbc, ld_x, proj, ld_p, dt_col0, (const TW*)dt_bias,         \
            (const TW*)a_log, (const TW*)d_skip, state, y, heads, groups, P, N, n_reqs, req_row_start, req_n_rows,      \
            req_state_slot, write_state, (vec && (((uintptr_t)state) & 15) == 0) ? 1 : 0)
#define KF_GO(TW)                                  \
  do {                                             \
    if (N <= 32) KF_STEP(1, TW);                   \
    else if (N <= 64) KF_STEP(2, TW);              \
    else if (N <= 128) KF_STEP(4, TW);             \
    else KF_STEP(8, TW);                           \
  } while (0)
    if (w_dtype == KF_F32) KF_GO(float);
    else KF_GO(__nv_bfloat16);
#undef KF_GO
#undef KF_STEP
  } else if (w_dtype == KF_F32) {
    ssm_launch_walk<float, false>(grid, stream, xbc, ld_x, proj, ld_p, dt_col0, dt_bias, a_log, d_skip, state, req_state_slot, state,
                                  req_state_slot, nullptr, y, heads, groups, P, N, n_reqs, req_row_start, req_n_rows, write_state, vec);
  } else {
    ssm_launch_walk<__nv_bfloat16, false>(grid, stream, xbc, ld_x, proj, ld_p, dt_col0, dt_bias, a_log, d_skip, state, req_state_slot,
                                          state, req_state_slot, nullptr, y, heads, groups, P, N, n_reqs, req_row_start, req_n_rows,
                                          write_state, vec);
  }
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// The same over chunks of `chunk_rows` rows walked side by side (see above).  Scratch from the caller: `tab`
// (5 * max_chunks + 2 * n_reqs ints), `chunk_state` (max_chunks * heads * P * N floats) and `chunk_decay`
// (max_chunks * heads floats), with max_chunks >= rows / chunk_rows + n_reqs.
KF_API int kf_ssm_scan_chunked(const float* xbc, int ld_x, const float* proj, int ld_p, int dt_col0, const void* dt_bias,
                               const void* a_log, const void* d_skip, int w_dtype, float* state, float* y, int heads,
                               int groups, int P, int N, int n_reqs, const int* req_row_start, const int* req_n_rows,
                               const int* req_state_slot, int write_state, int chunk_rows, int max_chunks, int* tab,
                               float* chunk_state, float* chunk_decay, cudaStream_t stream) {
  if (n_reqs <= 0) return KF_OK;
  if (N < 1 || N > SSM_MAX_N || P < 1 || heads < 1 || groups < 1 || heads % groups || chunk_rows < 1 || max_chunks < 1)
    return KF_ERR_SIZE;
  if (w_dtype != KF_F32 && w_dtype != KF_BF16) return KF_ERR_DTYPE;
  const int vec = (N % 4 == 0 && P % 4 == 0 && ld_x % 4 == 0 && ((uintptr_t)xbc & 15) == 0) ? 1 : 0;
  const int* c_row_start = tab;
  const int* c_n_rows = tab + max_chunks;
  const int* c_n_rows_a = tab + 2 * max_chunks;
  const int* c_ident = tab + 3 * max_chunks;
  const int* c_out_slot = tab + 4 * max_chunks;
  const int* r_chunk0 = tab + 5 * max_chunks;
  const int* r_nchunks = r_chunk0 + n_reqs;
  kf_launch(ssm_chunk_table_kernel, dim3(1), dim3(32), 0, stream, n_reqs, req_row_start, req_n_rows, req_state_slot, chunk_rows,
            max_chunks, tab);
  const dim3 grid(max_chunks * heads, kf_ceil_div(P, SSM_PC));
  if (w_dtype == KF_F32)
    ssm_launch_walk<float, true>(grid, stream, xbc, ld_x, proj, ld_p, dt_col0, dt_bias, a_log, d_skip, nullptr, c_ident, chunk_state,
                                 c_ident, chunk_decay, nullptr, heads, groups, P, N, max_chunks, c_row_start, c_n_rows_a, 1, vec);
  else
    ssm_launch_walk<__nv_bfloat16, true>(grid, stream, xbc, ld_x, proj, ld_p, dt_col0, dt_bias, a_log, d_skip, nullptr, c_ident,
                                         chunk_state, c_ident, chunk_decay, nullptr, heads, groups, P, N, max_chunks, c_row_start,
                                         c_n_rows_a, 1, vec);
  const int PN = P * N;
  kf_launch(ssm_chunk_fold_kernel, dim3(n_reqs, heads, kf_ceil_div(PN, 256)), dim3(256), 0, stream, (const float*)state, chunk_state,
            (const float*)chunk_decay, heads, PN, n_reqs, req_state_slot, r_chunk0, r_nchunks);
  if (w_dtype == KF_F32)
    ssm_launch_walk<float, false>(grid, stream, xbc, ld_x, proj, ld_p, dt_col0, dt_bias, a_log, d_skip, chunk_state, c_ident, state,
                                  c_out_slot, nullptr, y, heads, groups, P, N, max_chunks, c_row_start, c_n_rows, write_state, vec);
  else
    ssm_launch_walk<__nv_bfloat16, false>(grid, stream, xbc, ld_x, proj, ld_p, dt_col0, dt_bias, a_log, d_skip, chunk_state, c_ident,
                                          state, c_out_slot, nullptr, y, heads, groups, P, N, max_chunks, c_row_start, c_n_rows,
                                          write_state, vec);
  KF_CHECK_LAUNCH();
  return KF_OK;
}

// out[t][j] = rms_part(y[t] * silu(z[t]))[j] * w[j]: the gate is applied first, then every one of `parts` equal parts
// of the row is divided by its own root mean square (eps inside the root).  z is columns z_col0.. of a 32-bit matrix
// with ld columns.  One block per (row, part); sums in 32-bit; y and z are read once (a thread keeps its gated values).
template <typename TW, typename TO>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ z, int ld, int z_col0,
                                        const TW* __restrict__ w, float eps, int inner, int parts, TO* __restrict__ out,
                                        const int* __restrict__ row_req) {
  kf_pdl_trigger();
  kf_pdl_wait();
  __shared__ float red[33];
  constexpr int KEEP = 8;                                   // gated values a thread keeps between the two passes
  const int t = blockIdx.x, part = blockIdx.y;
  const int len = inner / parts, j0 = part * len;
  if (row_req[t] < 0) {
    for (int j = threadIdx.x; j < len; j += blockDim.x) kf_store(out, (size_t)t * inner + j0 + j, 0.f);
    return;
  }
  const float* yr = y + (size_t)t * inner + j0;
  const float* zr = z + (size_t)t * ld + z_col0 + j0;
  float v[KEEP];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < KEEP; ++c) {
    const int j = threadIdx.x + c * blockDim.x;
    v[c] = 0.f;
    if (j < len) {
      const float zz = zr[j];
      v[c] = yr[j] * (zz / (1.f + expf(-zz)));
      ss = fmaf(v[c], v[c], ss);
    }
  }
  for (int j = threadIdx.x + KEEP * blockDim.x; j < len; j += blockDim.x) {       // parts longer than KEEP per thread
    const float zz = zr[j];
    const float u = yr[j] * (zz / (1.f + expf(-zz)));
    ss = fmaf(u, u, ss);
  }
  ss = kf_block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / (float)len + eps);
#pragma unroll
  for (int c = 0; c < KEEP; ++c) {
    const int j = threadIdx.x + c * blockDim.x;
    if (j < len) kf_store(out, (size_t)t * inner + j0 + j, v[c] * inv * kf_load(w, j0 + j));
  }
  for (int j = threadIdx.x + KEEP * blockDim.x; j < len; j += blockDim.x) {
    const float zz = zr[j];
    const float u = yr[j] * (zz / (1.f + expf(-zz)));
    kf_store(out, (size_t)t * inner + j0 + j, u * inv * kf_load(w, j0 + j));
  }
}

KF_API int kf_gated_group_norm(const float* y, const float* z, int ld, int z_col0, const void* w, int w_dtype, float eps,
                               int inner, int parts, void* out, int out_dtype, const int* row_req, int T,
                               cudaStream_t stream) {
  if (T <= 0) return KF_OK;
  if (parts < 1 || inner % parts) return KF_ERR_SIZE;
  const int len = inner / parts;
  // few rows (decoding): as many threads as the part has groups of four; many rows: blocks of at most 512 threads
  const int threads = (len >= 4096 && T < 256) ? 1024 : (len >= 2048 ? 512 : (len >= 1024 ? 256 : 128));
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
