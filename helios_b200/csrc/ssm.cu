// A recurrent mixer with a matrix state per head and ONE decay per head and token (a
// selective state-space layer in its recurrent form).  Per token and head, with x [P] the
// head's input, B and C [N] shared by the heads of a group, dt = softplus(dt_raw + dt_bias)
// and a = exp(-exp(A_log) dt):
//
//   S <- a S + dt B x^T        (S is [N, P])
//   y  = S^T C + D x
//
// The columns of S never mix: a quad of threads owns one column (a quarter of its N rows
// each, in registers) and walks the request's tokens in order from the state the request's
// slot holds, so a request's numbers do not depend on how its tokens were cut into steps or
// on the rest of the batch.  State, step sizes, decays and the recurrence are float32.
//
// Kernels: `ssm_scan` (the recurrence) and `gated_group_rmsnorm` (y * silu(z), then an RMS
// norm in equal parts of the row, times a weight per channel).
#include "common.cuh"

constexpr int SSM_CHUNK = 16;       // tokens staged in shared memory at a time
constexpr int SSM_COLS = 32;        // columns of S a block owns (a quad of threads each)

// xbc [T, ld]: x at x_off + h * P, B at b_off + g * N, C at c_off + g * N (after the short
// convolution and silu); dt_raw [T, dt_ld] at column h.  state of a slot: [heads, N, P].
template <typename T, int ROWS>
__global__ void __launch_bounds__(SSM_COLS * 4)
ssm_scan_kernel(float* __restrict__ y, const T* __restrict__ xbc, int ld, int x_off, int b_off, int c_off,
                const T* __restrict__ dt_raw, int dt_ld, const float* __restrict__ a_log,
                const float* __restrict__ dt_bias, const float* __restrict__ d_skip,
                float* __restrict__ state, long state_stride, const int* __restrict__ cu_tokens,
                const int* __restrict__ slots, int heads, int groups, int N, int P) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* Bs = sm;                              // [SSM_CHUNK][N]
  float* Cs = Bs + SSM_CHUNK * N;              // [SSM_CHUNK][N]
  float* xs = Cs + SSM_CHUNK * N;              // [SSM_CHUNK][SSM_COLS]
  float* dts = xs + SSM_CHUNK * SSM_COLS;      // [SSM_CHUNK]
  float* as = dts + SSM_CHUNK;                 // [SSM_CHUNK]
  const int h = blockIdx.y, seq = blockIdx.z;
  const int g = h / (heads / groups);
  const int col0 = blockIdx.x * SSM_COLS;
  const int quad = threadIdx.x >> 2, part = threadIdx.x & 3;
  const int col = col0 + quad;
  const bool live = col < P;
  const int t0 = cu_tokens[seq], t1 = cu_tokens[seq + 1];
  float* S = state + (size_t)slots[seq] * state_stride + (size_t)h * N * P;
  float s[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int n = part + 4 * i;
    s[i] = (live && n < N) ? S[(size_t)n * P + col] : 0.f;
  }
  const float neg_rate = -expf(a_log[h]);
  const float bias = dt_bias[h], skip = d_skip[h];
  for (int c0 = t0; c0 < t1; c0 += SSM_CHUNK) {
    const int n_tok = min(SSM_CHUNK, t1 - c0);
    __syncthreads();
    for (int i = threadIdx.x; i < n_tok * N; i += blockDim.x) {
      const int j = i / N, n = i - j * N;
      const T* r = xbc + (size_t)(c0 + j) * ld;
      Bs[j * N + n] = to_float(r[b_off + g * N + n]);
      Cs[j * N + n] = to_float(r[c_off + g * N + n]);
    }
    for (int i = threadIdx.x; i < n_tok * SSM_COLS; i += blockDim.x) {
      const int j = i / SSM_COLS, c = i - j * SSM_COLS;
      xs[i] = (col0 + c < P) ? to_float(xbc[(size_t)(c0 + j) * ld + x_off + h * P + col0 + c]) : 0.f;
    }
    if (threadIdx.x < n_tok) {
      const float v = to_float(dt_raw[(size_t)(c0 + threadIdx.x) * dt_ld + h]) + bias;
      const float dt = fmaxf(v, 0.f) + log1pf(expf(-fabsf(v)));      // softplus, no clamp
      dts[threadIdx.x] = dt;
      as[threadIdx.x] = expf(neg_rate * dt);
    }
    __syncthreads();
    for (int j = 0; j < n_tok; ++j) {
      const float a = as[j], xv = xs[j * SSM_COLS + quad];
      const float dx = dts[j] * xv;
      const float* Bj = Bs + j * N;
      const float* Cj = Cs + j * N;
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int i = 0; i < ROWS; ++i) {
        const int n = part + 4 * i;
        if (n < N) {
          s[i] = fmaf(a, s[i], dx * Bj[n]);
          if (i & 1) acc1 = fmaf(s[i], Cj[n], acc1); else acc0 = fmaf(s[i], Cj[n], acc0);
        }
      }
      float acc = acc0 + acc1;
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (live && part == 0) y[(size_t)(c0 + j) * heads * P + (size_t)h * P + col] = fmaf(skip, xv, acc);
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int n = part + 4 * i;
    if (live && n < N) S[(size_t)n * P + col] = s[i];
  }
}

HB_EXPORT int hb_ssm_scan(float* y, const void* xbc, int ld, int x_off, int b_off, int c_off,
                          const void* dt_raw, int dt_ld, const float* a_log, const float* dt_bias,
                          const float* d_skip, float* state, long state_stride, const int* cu_tokens,
                          const int* slots, int n_tokens, int n_seqs, int heads, int groups, int N, int P,
                          int act_dt, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return HB_OK;
  if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || N > 256 || P <= 0) return HB_BAD_ARGUMENT;
  const size_t smem = (size_t)(2 * SSM_CHUNK * N + SSM_CHUNK * SSM_COLS + 2 * SSM_CHUNK) * sizeof(float);
  const dim3 grid((P + SSM_COLS - 1) / SSM_COLS, heads, n_seqs);
#define HB_SSM(R)                                                                                   \
  hb_launch(ssm_scan_kernel<TA, R>, grid, dim3(SSM_COLS * 4), smem, stream, y, (const TA*)xbc, ld,  \
            x_off, b_off, c_off, (const TA*)dt_raw, dt_ld, a_log, dt_bias, d_skip, state,           \
            state_stride, cu_tokens, slots, heads, groups, N, P)
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (N <= 16) HB_SSM(4);
    else if (N <= 32) HB_SSM(8);
    else if (N <= 64) HB_SSM(16);
    else if (N <= 128) HB_SSM(32);
    else HB_SSM(64));
#undef HB_SSM
  return hb_check_launch();
}

// out[t, c] = v[c] * rsqrt(mean over c's part of v^2 + eps) * w[c],  v = y[t, c] * silu(z[t, c]):
// the gate comes before the norm, and the row is normed in `parts` equal parts, each by its
// own root mean square.  y float32 [T, inner]; z [T, >= inner] rows z_ld apart; one warp per
// (token, part); float32 arithmetic.
template <typename T>
__global__ void __launch_bounds__(128)
gated_group_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ z,
                           int z_ld, const float* __restrict__ w, int n_tokens, int inner, int parts,
                           float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (long)n_tokens * parts) return;
  const int t = (int)(item / parts), p = (int)(item - (long)t * parts);
  const int size = inner / parts;
  const float* yr = y + (size_t)t * inner + (size_t)p * size;
  const T* zr = z + (size_t)t * z_ld + (size_t)p * size;
  float ss = 0.f;
  for (int c = lane; c < size; c += 32) {
    const float g = to_float(zr[c]);
    const float v = yr[c] * (g / (1.f + expf(-g)));
    ss = fmaf(v, v, ss);
  }
  const float f = rsqrtf(warp_sum(ss) / (float)size + eps);
  T* o = out + (size_t)t * inner + (size_t)p * size;
  const float* wr = w + (size_t)p * size;
  for (int c = lane; c < size; c += 32) {
    const float g = to_float(zr[c]);
    const float v = yr[c] * (g / (1.f + expf(-g)));
    o[c] = from_float<T>(v * f * wr[c]);
  }
}

HB_EXPORT int hb_gated_group_rmsnorm(void* out, const float* y, const void* z, int z_ld, const float* w,
                                     int n_tokens, int inner, int parts, float eps, int act_dt,
                                     cudaStream_t stream) {
  if (n_tokens <= 0) return HB_OK;
  if (inner <= 0 || parts <= 0 || inner % parts || z_ld < inner) return HB_BAD_ARGUMENT;
  const long items = (long)n_tokens * parts;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(gated_group_rmsnorm_kernel<TA>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream,
              (TA*)out, y, (const TA*)z, z_ld, w, n_tokens, inner, parts, eps));
  return hb_check_launch();
}
