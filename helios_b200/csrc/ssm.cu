// A recurrent mixer with a matrix state per head and ONE decay per head and token (a
// selective state-space layer in its recurrent form).  Per token and head, with x [P] the
// head's input, B and C [N] shared by the heads of a group, dt = softplus(dt_raw + dt_bias)
// and a = exp(-exp(A_log) dt):
//
//   S <- a S + dt B x^T        (S is [N, P])
//   y  = S^T C + D x
//
// The columns of S never mix: a group of 4 or 8 threads owns one column (a share of its N
// rows each, in registers; neighbouring lanes in the kernel for portions, the same lane of 4 or
// 8 warps in the kernel for single tokens) and walks the request's tokens in order from the
// state the request's slot holds, so a request's numbers do not depend on how its tokens were cut into steps or
// on the rest of the batch.  State, step sizes, decays and the recurrence are float32.
//
// Kernels: `ssm_scan` (the recurrence, for steps of few tokens a request), `ssm_stage` +
// `ssm_scan_staged` (the same recurrence for portions of prompts: inputs laid out once, in
// parallel over tokens, then fetched a chunk ahead of the scan) and `gated_group_rmsnorm`
// (y * silu(z), then an RMS norm in equal parts of the row, times a weight per channel).
#include "common.cuh"

constexpr int SSM_CHUNK = 16;       // tokens staged in shared memory at a time
constexpr int SSM_COLS = 32;        // columns of S a block owns (PARTS threads each)

// One thread's share of one token of one column.  PARTS (4 or 8) threads share a column: thread `part`
// owns the rows 4 (part + PARTS k) + e (k < ROWS / 4, e < 4): groups of four consecutive rows,
// dealt round the threads, so that they read consecutive 16-byte pieces of B and of C.  Bj and
// Cj hold PARTS x ROWS floats (zeros beyond the state's rows, which keeps those entries of s at
// zero).  Both scan kernels go through here, so a token's numbers do not depend on which ran.
template <int ROWS, int PARTS>
__device__ __forceinline__ float ssm_token_share(float (&s)[ROWS], const float* __restrict__ Bj,
                                           const float* __restrict__ Cj, float a, float dx, int part) {
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int k = 0; k < ROWS / 4; ++k) {
    const float4 b = *reinterpret_cast<const float4*>(Bj + 4 * (part + PARTS * k));
    const float4 c = *reinterpret_cast<const float4*>(Cj + 4 * (part + PARTS * k));
    s[4 * k + 0] = fmaf(a, s[4 * k + 0], dx * b.x);
    s[4 * k + 1] = fmaf(a, s[4 * k + 1], dx * b.y);
    s[4 * k + 2] = fmaf(a, s[4 * k + 2], dx * b.z);
    s[4 * k + 3] = fmaf(a, s[4 * k + 3], dx * b.w);
    acc[0] = fmaf(s[4 * k + 0], c.x, acc[0]);
    acc[1] = fmaf(s[4 * k + 1], c.y, acc[1]);
    acc[2] = fmaf(s[4 * k + 2], c.z, acc[2]);
    acc[3] = fmaf(s[4 * k + 3], c.w, acc[3]);
  }
  return (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

// The read-out of a column is the sum of its threads' shares in the order of a butterfly:
// ((r0 + r1) + (r2 + r3)) + ((r4 + r5) + (r6 + r7)).  The kernel for portions has the shares in
// neighbouring lanes, the kernel for single tokens in shared memory; both add in this order.
template <int PARTS>
__device__ __forceinline__ float ssm_sum_lanes(float r) {
  r += __shfl_xor_sync(0xffffffffu, r, 1);
  r += __shfl_xor_sync(0xffffffffu, r, 2);
  if (PARTS == 8) r += __shfl_xor_sync(0xffffffffu, r, 4);
  return r;
}

template <int PARTS>
__device__ __forceinline__ float ssm_sum_shared(const float* __restrict__ r, int stride) {
  float lo = (r[0] + r[stride]) + (r[2 * stride] + r[3 * stride]);
  if (PARTS == 8) lo += (r[4 * stride] + r[5 * stride]) + (r[6 * stride] + r[7 * stride]);
  return lo;
}

template <int PARTS>
__device__ __forceinline__ int ssm_row(int part, int i) { return 4 * (part + PARTS * (i >> 2)) + (i & 3); }

__device__ __forceinline__ float ssm_softplus(float v) { return fmaxf(v, 0.f) + log1pf(expf(-fabsf(v))); }

// Steps of few tokens a request (decoding): inputs are read where the convolution left them.
// xbc [T, ld]: x at x_off + h * P, B at b_off + g * N, C at c_off + g * N (after the short
// convolution and silu); dt_raw [T, dt_ld] at column h.  state of a slot: [heads, N, P].
template <typename T, int ROWS, int PARTS>
__global__ void __launch_bounds__(SSM_COLS * PARTS, ROWS <= 8 ? 1024 / (SSM_COLS * PARTS) : ROWS <= 16 ? 3 : 1)
ssm_scan_kernel(float* __restrict__ y, const T* __restrict__ xbc, int ld, int x_off, int b_off, int c_off,
                const T* __restrict__ dt_raw, int dt_ld, const float* __restrict__ a_log,
                const float* __restrict__ dt_bias, const float* __restrict__ d_skip,
                float* __restrict__ state, long state_stride, const int* __restrict__ cu_tokens,
                const int* __restrict__ slots, int heads, int groups, int N, int P) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int NP = PARTS * ROWS;
  extern __shared__ __align__(16) float sm[];
  float* Bs = sm;                              // [SSM_CHUNK][NP]
  float* Cs = Bs + SSM_CHUNK * NP;             // [SSM_CHUNK][NP]
  float* xs = Cs + SSM_CHUNK * NP;             // [SSM_CHUNK][SSM_COLS]
  float* dts = xs + SSM_CHUNK * SSM_COLS;      // [SSM_CHUNK]
  float* as = dts + SSM_CHUNK;                 // [SSM_CHUNK]
  float* shares = as + SSM_CHUNK;              // [2][PARTS][SSM_COLS]: the tokens take turns
  const int h = blockIdx.y, seq = blockIdx.z;
  const int g = h / (heads / groups);
  const int col0 = blockIdx.x * SSM_COLS;
  // a lane a column, a warp a share of the rows: the state, which is most of what a step of
  // single tokens moves, is read and written as whole rows of 32 columns
  const int quad = threadIdx.x & 31, part = threadIdx.x >> 5;
  const int col = col0 + quad;
  const bool live = col < P;
  const int t0 = cu_tokens[seq], t1 = cu_tokens[seq + 1];
  float* S = state + (size_t)slots[seq] * state_stride + (size_t)h * N * P;
  float s[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int n = ssm_row<PARTS>(part, i);
    s[i] = (live && n < N) ? S[(size_t)n * P + col] : 0.f;
  }
  int turn = 0;
  const float neg_rate = -expf(a_log[h]);
  const float bias = dt_bias[h], skip = d_skip[h];
  for (int c0 = t0; c0 < t1; c0 += SSM_CHUNK) {
    const int n_tok = min(SSM_CHUNK, t1 - c0);
    __syncthreads();
    for (int i = threadIdx.x; i < n_tok * NP; i += blockDim.x) {
      const int j = i / NP, n = i - j * NP;
      const T* r = xbc + (size_t)(c0 + j) * ld;
      Bs[i] = n < N ? to_float(r[b_off + g * N + n]) : 0.f;
      Cs[i] = n < N ? to_float(r[c_off + g * N + n]) : 0.f;
    }
    for (int i = threadIdx.x; i < n_tok * SSM_COLS; i += blockDim.x) {
      const int j = i / SSM_COLS, c = i - j * SSM_COLS;
      xs[i] = (col0 + c < P) ? to_float(xbc[(size_t)(c0 + j) * ld + x_off + h * P + col0 + c]) : 0.f;
    }
    if (threadIdx.x < n_tok) {
      const float dt = ssm_softplus(to_float(dt_raw[(size_t)(c0 + threadIdx.x) * dt_ld + h]) + bias);   // no clamp
      dts[threadIdx.x] = dt;
      as[threadIdx.x] = expf(neg_rate * dt);
    }
    __syncthreads();
    for (int j = 0; j < n_tok; ++j) {
      const float xv = xs[j * SSM_COLS + quad];
      float* mine = shares + turn * PARTS * SSM_COLS;
      mine[part * SSM_COLS + quad] = ssm_token_share<ROWS, PARTS>(s, Bs + j * NP, Cs + j * NP, as[j], dts[j] * xv, part);
      __syncthreads();
      if (live && part == 0)
        y[(size_t)(c0 + j) * heads * P + (size_t)h * P + col] = fmaf(skip, xv, ssm_sum_shared<PARTS>(mine + quad, SSM_COLS));
      turn ^= 1;
    }
  }
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int n = ssm_row<PARTS>(part, i);
    if (live && n < N) S[(size_t)n * P + col] = s[i];
  }
}

// Steps with portions of prompts.  `ssm_stage` (parallel over tokens) first lays the scan's
// inputs out as float32 rows that copy in 16-byte pieces whatever the sizes:
//   bc [T, groups, 2 NP]   B then C, NP = PARTS x ROWS floats each, zeros beyond N
//   xs [T, heads, PP]      x, PP = P rounded up to whole blocks of SSM_COLS columns, zeros beyond P
//   da [T, heads, 2]       dt = softplus(dt_raw + dt_bias) and the decay exp(-exp(A_log) dt)
template <typename T>
__global__ void __launch_bounds__(256)
ssm_stage_kernel(float* __restrict__ bc, float* __restrict__ xs, float* __restrict__ da,
                 const T* __restrict__ xbc, int ld, int x_off, int b_off, int c_off,
                 const T* __restrict__ dt_raw, int dt_ld, const float* __restrict__ a_log,
                 const float* __restrict__ dt_bias, int heads, int groups, int N, int P, int NP, int PP) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const T* r = xbc + (size_t)t * ld;
  const int n_bc = groups * 2 * NP, n_x = heads * PP;
  for (int i = threadIdx.x; i < n_bc; i += blockDim.x) {
    const int g = i / (2 * NP), rest = i - g * 2 * NP;
    const int which = rest / NP, n = rest - which * NP;
    bc[(size_t)t * n_bc + i] = n < N ? to_float(r[(which ? c_off : b_off) + g * N + n]) : 0.f;
  }
  for (int i = threadIdx.x; i < n_x; i += blockDim.x) {
    const int h = i / PP, c = i - h * PP;
    xs[(size_t)t * n_x + i] = c < P ? to_float(r[x_off + h * P + c]) : 0.f;
  }
  for (int h = threadIdx.x; h < heads; h += blockDim.x) {
    const float dt = ssm_softplus(to_float(dt_raw[(size_t)t * dt_ld + h]) + dt_bias[h]);
    da[((size_t)t * heads + h) * 2] = dt;
    da[((size_t)t * heads + h) * 2 + 1] = expf(-expf(a_log[h]) * dt);
  }
}

__device__ __forceinline__ void ssm_cp16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)),
               "l"(gmem));
}
__device__ __forceinline__ void ssm_cp8(void* smem, const void* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)),
               "l"(gmem));
}

// The scan over staged rows: chunks of SSM_CHUNK tokens arrive by cp.async one chunk ahead of
// the one being computed; a chunk's outputs leave through shared memory as whole rows.  A block
// owns COLS (16 or 32) columns; a column's numbers do not depend on which.
template <int ROWS, int PARTS, int COLS>
__global__ void __launch_bounds__(COLS * PARTS)
ssm_scan_staged_kernel(float* __restrict__ y, const float* __restrict__ bc, const float* __restrict__ xst,
                       const float* __restrict__ da, const float* __restrict__ d_skip,
                       float* __restrict__ state, long state_stride, const int* __restrict__ cu_tokens,
                       const int* __restrict__ slots, int heads, int groups, int N, int P, int PP) {
  constexpr int NP = PARTS * ROWS;
  constexpr int STAGE = SSM_CHUNK * (2 * NP + COLS + 2);     // floats a stage
  extern __shared__ __align__(16) float sm[];
  float* ys = sm + 2 * STAGE;                  // [SSM_CHUNK][COLS]
  const int h = blockIdx.y, seq = blockIdx.z;
  const int g = h / (heads / groups);
  const int col0 = blockIdx.x * COLS;
  const int quad = threadIdx.x / PARTS, part = threadIdx.x % PARTS;
  const int col = col0 + quad;
  const bool live = col < P;
  const int t0 = cu_tokens[seq], t1 = cu_tokens[seq + 1];
  float* S = state + (size_t)slots[seq] * state_stride + (size_t)h * N * P;
  float s[ROWS];
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int n = ssm_row<PARTS>(part, i);
    s[i] = (live && n < N) ? S[(size_t)n * P + col] : 0.f;
  }
  const float skip = d_skip[h];
  auto fetch = [&](int c0, int stage) {
    const int n_tok = min(SSM_CHUNK, t1 - c0);
    float* bcs = sm + stage * STAGE;                       // [SSM_CHUNK][2 NP]
    float* xs = bcs + SSM_CHUNK * 2 * NP;                  // [SSM_CHUNK][COLS]
    float* das = xs + SSM_CHUNK * COLS;                // [SSM_CHUNK][2]
    constexpr int V_BC = 2 * NP / 4, V_X = COLS / 4;
    for (int i = threadIdx.x; i < n_tok * V_BC; i += blockDim.x) {
      const int j = i / V_BC, v = i - j * V_BC;
      ssm_cp16(bcs + j * 2 * NP + v * 4, bc + ((size_t)(c0 + j) * groups + g) * 2 * NP + v * 4);
    }
    for (int i = threadIdx.x; i < n_tok * V_X; i += blockDim.x) {
      const int j = i / V_X, v = i - j * V_X;
      ssm_cp16(xs + j * COLS + v * 4, xst + ((size_t)(c0 + j) * heads + h) * PP + col0 + v * 4);
    }
    if (threadIdx.x < n_tok) ssm_cp8(das + threadIdx.x * 2, da + ((size_t)(c0 + threadIdx.x) * heads + h) * 2);
  };
  if (t0 < t1) fetch(t0, 0);
  asm volatile("cp.async.commit_group;\n" ::);
  int stage = 0;
  for (int c0 = t0; c0 < t1; c0 += SSM_CHUNK, stage ^= 1) {
    const int n_tok = min(SSM_CHUNK, t1 - c0);
    if (c0 + SSM_CHUNK < t1) fetch(c0 + SSM_CHUNK, stage ^ 1);
    asm volatile("cp.async.commit_group;\n" ::);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    const float* bcs = sm + stage * STAGE;
    const float* xs = bcs + SSM_CHUNK * 2 * NP;
    const float* das = xs + SSM_CHUNK * COLS;
    auto share = [&](int j, float& xv) {
      xv = xs[j * COLS + quad];
      const float2 d = *reinterpret_cast<const float2*>(das + 2 * j);
      return ssm_token_share<ROWS, PARTS>(s, bcs + j * 2 * NP, bcs + j * 2 * NP + NP, d.y, d.x * xv, part);
    };
    if (n_tok == SSM_CHUNK) {
      // whole chunks four tokens at a time: only the state's update chains one token to the
      // next, so the four tokens' loads come first and their read-outs' sums and shuffles
      // overlap; the outputs are stored after the four (a store to shared memory between two
      // tokens would keep the next token's loads behind it)
      constexpr int GROUP = 4;
#pragma unroll 1
      for (int j0 = 0; j0 < SSM_CHUNK; j0 += GROUP) {
        float r[GROUP], xv[GROUP];
#pragma unroll
        for (int u = 0; u < GROUP; ++u) r[u] = share(j0 + u, xv[u]);
#pragma unroll
        for (int u = 0; u < GROUP; ++u) r[u] = ssm_sum_lanes<PARTS>(r[u]);
        if (part == 0) {
#pragma unroll
          for (int u = 0; u < GROUP; ++u) ys[(j0 + u) * COLS + quad] = fmaf(skip, xv[u], r[u]);
        }
      }
    } else {
      for (int j = 0; j < n_tok; ++j) {
        float xv;
        const float r = ssm_sum_lanes<PARTS>(share(j, xv));
        if (part == 0) ys[j * COLS + quad] = fmaf(skip, xv, r);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n_tok * COLS; i += blockDim.x) {
      const int j = i / COLS, c = i - j * COLS;
      if (col0 + c < P) y[(size_t)(c0 + j) * heads * P + (size_t)h * P + col0 + c] = ys[i];
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    const int n = ssm_row<PARTS>(part, i);
    if (live && n < N) S[(size_t)n * P + col] = s[i];
  }
}

// Floats a padded row of B or C takes: PARTS x ROWS, with 4 threads a column up to 32 state
// rows and 8 beyond (more warps an SM to hide the loads of B and C, fewer rows a thread).
static inline int ssm_padded_rows(int N) { return N <= 16 ? 16 : N <= 32 ? 32 : N <= 64 ? 64 : N <= 128 ? 128 : 256; }

HB_EXPORT int hb_ssm_scan(float* y, const void* xbc, int ld, int x_off, int b_off, int c_off,
                          const void* dt_raw, int dt_ld, const float* a_log, const float* dt_bias,
                          const float* d_skip, float* state, long state_stride, const int* cu_tokens,
                          const int* slots, int n_tokens, int n_seqs, int heads, int groups, int N, int P,
                          int act_dt, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return HB_OK;
  if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || N > 256 || P <= 0) return HB_BAD_ARGUMENT;
  const int NP = ssm_padded_rows(N);
  const size_t smem = (size_t)(2 * SSM_CHUNK * NP + SSM_CHUNK * SSM_COLS + 2 * SSM_CHUNK + 2 * 8 * SSM_COLS) * sizeof(float);
  const dim3 grid((P + SSM_COLS - 1) / SSM_COLS, heads, n_seqs);
#define HB_SSM(R, PT)                                                                               \
  hb_launch(ssm_scan_kernel<TA, R, PT>, grid, dim3(SSM_COLS * PT), smem, stream, y, (const TA*)xbc, \
            ld, x_off, b_off, c_off, (const TA*)dt_raw, dt_ld, a_log, dt_bias, d_skip, state,       \
            state_stride, cu_tokens, slots, heads, groups, N, P)
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (NP == 16) HB_SSM(4, 4);
    else if (NP == 32) HB_SSM(8, 4);
    else if (NP == 64) HB_SSM(8, 8);
    else if (NP == 128) HB_SSM(16, 8);
    else HB_SSM(32, 8));
#undef HB_SSM
  return hb_check_launch();
}

// Floats the staged rows of a token take: bc, xs, da (see ssm_stage_kernel).
HB_EXPORT int hb_ssm_stage_sizes(int heads, int groups, int N, int P, int* bc, int* xs, int* da) {
  if (heads <= 0 || groups <= 0 || N <= 0 || N > 256 || P <= 0) return HB_BAD_ARGUMENT;
  *bc = groups * 2 * ssm_padded_rows(N);
  *xs = heads * ((P + SSM_COLS - 1) / SSM_COLS) * SSM_COLS;
  *da = heads * 2;
  return HB_OK;
}

template <int ROWS, int PARTS, int COLS>
static int ssm_launch_staged_cols(float* y, const float* bc, const float* xs, const float* da, const float* d_skip,
                             float* state, long state_stride, const int* cu_tokens, const int* slots,
                             int n_seqs, int heads, int groups, int N, int P, int PP, cudaStream_t stream) {
  constexpr int NP = PARTS * ROWS;
  const size_t smem = (size_t)(2 * SSM_CHUNK * (2 * NP + COLS + 2) + SSM_CHUNK * COLS) * sizeof(float);
  static bool raised = false;
  if (smem > 48 * 1024 && !raised) {
    if (cudaFuncSetAttribute(ssm_scan_staged_kernel<ROWS, PARTS, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
      return HB_LAUNCH_FAILED;
    raised = true;
  }
  // a plain launch: started while the kernel before it still fills the SMs, the scan's few
  // long-lived blocks would share SMs with it for their whole life
  ssm_scan_staged_kernel<ROWS, PARTS, COLS><<<dim3(PP / COLS, heads, n_seqs), dim3(COLS * PARTS), smem, stream>>>(
      y, bc, xs, da, d_skip, state, state_stride, cu_tokens, slots, heads, groups, N, P, PP);
  return hb_check_launch();
}

static int ssm_sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
      v = 148;
    n = v;
  }
  return n;
}

// Blocks of 32 columns, or of 16 where those would leave SMs without a block (one long prompt):
// the scan's time is its tokens times a warp's time a token, whatever a block's width.
template <int ROWS, int PARTS>
static int ssm_launch_staged(float* y, const float* bc, const float* xs, const float* da, const float* d_skip,
                             float* state, long state_stride, const int* cu_tokens, const int* slots,
                             int n_seqs, int heads, int groups, int N, int P, int PP, cudaStream_t stream) {
  if ((long)(PP / SSM_COLS) * heads * n_seqs < ssm_sm_count())
    return ssm_launch_staged_cols<ROWS, PARTS, SSM_COLS / 2>(y, bc, xs, da, d_skip, state, state_stride, cu_tokens,
                                                             slots, n_seqs, heads, groups, N, P, PP, stream);
  return ssm_launch_staged_cols<ROWS, PARTS, SSM_COLS>(y, bc, xs, da, d_skip, state, state_stride, cu_tokens,
                                                       slots, n_seqs, heads, groups, N, P, PP, stream);
}

// The scan for steps with portions of prompts: stage (into bc / xs / da, float32 buffers of
// n_tokens x the sizes hb_ssm_stage_sizes gives), then scan.
HB_EXPORT int hb_ssm_scan_staged(float* y, float* bc, float* xs, float* da, const void* xbc, int ld, int x_off,
                                 int b_off, int c_off, const void* dt_raw, int dt_ld, const float* a_log,
                                 const float* dt_bias, const float* d_skip, float* state, long state_stride,
                                 const int* cu_tokens, const int* slots, int n_tokens, int n_seqs, int heads,
                                 int groups, int N, int P, int act_dt, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return HB_OK;
  if (heads <= 0 || groups <= 0 || heads % groups || N <= 0 || N > 256 || P <= 0) return HB_BAD_ARGUMENT;
  const int NP = ssm_padded_rows(N);
  const int PP = (P + SSM_COLS - 1) / SSM_COLS * SSM_COLS;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(ssm_stage_kernel<TA>, dim3(n_tokens), dim3(256), 0, stream, bc, xs, da, (const TA*)xbc, ld,
              x_off, b_off, c_off, (const TA*)dt_raw, dt_ld, a_log, dt_bias, heads, groups, N, P, NP, PP));
  const int st = hb_check_launch();
  if (st != HB_OK) return st;
#define HB_SSM(R, PT) return ssm_launch_staged<R, PT>(y, bc, xs, da, d_skip, state, state_stride, cu_tokens, \
                                                      slots, n_seqs, heads, groups, N, P, PP, stream)
  if (NP == 16) HB_SSM(4, 4);
  if (NP == 32) HB_SSM(8, 4);
  if (NP == 64) HB_SSM(8, 8);
  if (NP == 128) HB_SSM(16, 8);
  HB_SSM(32, 8);
#undef HB_SSM
}

// out[t, c] = v[c] * rsqrt(mean over c's part of v^2 + eps) * w[c],  v = y[t, c] * silu(z[t, c]):
// the gate comes before the norm, and the row is normed in `parts` equal parts, each by its
// own root mean square.  y float32 [T, inner]; z [T, >= inner] rows z_ld apart; one block per
// (token, part), whose gated values wait in registers between the sum and the output (up to
// GGN_PER_THREAD a thread; longer parts compute them twice); float32 arithmetic.  The order of
// the sum depends on the part's size and the block's alone.
constexpr int GGN_PER_THREAD = 16;

template <typename T, int THREADS>
__global__ void __launch_bounds__(THREADS)
gated_group_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ y, const T* __restrict__ z,
                           int z_ld, const float* __restrict__ w, int inner, int parts, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[THREADS / 32];
  const int t = blockIdx.x / parts, p = blockIdx.x - t * parts;
  const int size = inner / parts;
  const float* yr = y + (size_t)t * inner + (size_t)p * size;
  const T* zr = z + (size_t)t * z_ld + (size_t)p * size;
  const bool kept = size <= THREADS * GGN_PER_THREAD;
  float v[GGN_PER_THREAD];
  float ss = 0.f;
  if (kept) {
#pragma unroll
    for (int i = 0; i < GGN_PER_THREAD; ++i) {
      const int c = threadIdx.x + i * THREADS;
      v[i] = 0.f;
      if (c < size) {
        const float g = to_float(zr[c]);
        v[i] = yr[c] * (g / (1.f + expf(-g)));
      }
      ss = fmaf(v[i], v[i], ss);
    }
  } else {
    for (int c = threadIdx.x; c < size; c += THREADS) {
      const float g = to_float(zr[c]);
      const float x = yr[c] * (g / (1.f + expf(-g)));
      ss = fmaf(x, x, ss);
    }
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) scratch[threadIdx.x >> 5] = ss;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int i = 0; i < THREADS / 32; ++i) total += scratch[i];
  const float f = rsqrtf(total / (float)size + eps);
  T* o = out + (size_t)t * inner + (size_t)p * size;
  const float* wr = w + (size_t)p * size;
  if (kept) {
#pragma unroll
    for (int i = 0; i < GGN_PER_THREAD; ++i) {
      const int c = threadIdx.x + i * THREADS;
      if (c < size) o[c] = from_float<T>(v[i] * f * wr[c]);
    }
  } else {
    for (int c = threadIdx.x; c < size; c += THREADS) {
      const float g = to_float(zr[c]);
      const float x = yr[c] * (g / (1.f + expf(-g)));
      o[c] = from_float<T>(x * f * wr[c]);
    }
  }
}

HB_EXPORT int hb_gated_group_rmsnorm(void* out, const float* y, const void* z, int z_ld, const float* w,
                                     int n_tokens, int inner, int parts, float eps, int act_dt,
                                     cudaStream_t stream) {
  if (n_tokens <= 0) return HB_OK;
  if (inner <= 0 || parts <= 0 || inner % parts || z_ld < inner) return HB_BAD_ARGUMENT;
  const long items = (long)n_tokens * parts;
  const int size = inner / parts;
#define HB_GGN(TH)                                                                                 \
  hb_launch(gated_group_rmsnorm_kernel<TA, TH>, dim3((unsigned)items), dim3(TH), 0, stream, (TA*)out, y, \
            (const TA*)z, z_ld, w, inner, parts, eps)
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (size <= 128) HB_GGN(32);
    else if (size <= 1024) HB_GGN(128);
    else HB_GGN(256));
#undef HB_GGN
  return hb_check_launch();
}
