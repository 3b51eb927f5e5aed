// A recurrent mixer with a matrix state per head, written by the gated delta rule with one
// decay per key channel.  Per token and head (k, q unit vectors, q also times dk^-1/2):
//
//   S <- g (.) S            (g in (0,1)^dk scales the rows of S [dk, dv])
//   u  = beta (v - S^T k)
//   S <- S + k u^T
//   o  = S^T q              (the read-out sees this token's write)
//
// The columns of S never mix: a thread owns one column (dk values in registers) and walks
// the request's tokens in order, so a request's numbers do not depend on how its tokens
// were cut into steps or on the rest of the batch.  State, decays, gates, unit norms and
// the recurrence are float32.
//
// Kernels: `causal_conv_silu` (short causal convolution over time per channel + silu, the
// taps - 1 inputs before a step's first token taken from the request's slot),
// `causal_conv_state` (leaves the last taps - 1 inputs in the slot), `delta_prepare` and
// `delta_rule` (the recurrence) and `gated_rmsnorm` (o / rms(o) * weight * sigmoid(gate) per head).
#include "common.cuh"

// ---------------------------------------------------------------- short convolution
// x [T, ld] (the first `channels` columns), w [channels, taps] (the last column is the
// current token's), bias [channels] or null, conv state of a slot at state + slot * state_stride: [channels, taps - 1],
// oldest first.  out [T, channels].
template <typename T>
__global__ void causal_conv_silu_kernel(T* __restrict__ out, const T* __restrict__ x, int ld,
                                        const float* __restrict__ w, const float* __restrict__ bias,
                                        const float* __restrict__ state,
                                        long state_stride, const int* __restrict__ seq_of_token,
                                        const int* __restrict__ cu_tokens,
                                        const int* __restrict__ slots, int n_tokens, int channels,
                                        int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t total = (size_t)n_tokens * channels;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / channels), c = (int)(idx - (size_t)t * channels);
    const int s = seq_of_token[t];
    const int local = t - cu_tokens[s];
    const float* st = state + (size_t)slots[s] * state_stride + (size_t)c * (taps - 1);
    float acc = bias ? bias[c] : 0.f;
    for (int j = 0; j < taps; ++j) {
      const int src = local - (taps - 1) + j;
      const float v = src >= 0 ? to_float(x[(size_t)(t - (taps - 1) + j) * ld + c])
                               : st[(taps - 1) + src];
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
    }
    out[idx] = from_float<T>(acc / (1.f + expf(-acc)));
  }
}

// The same for bfloat16 rows that come in 16-byte pieces (channels, row stride and addresses
// multiples of eight values) and 2 to 4 taps: a thread takes eight neighbouring channels of
// CONV_TOKENS consecutive tokens, so that the channels' weights (16-byte loads) and the rows
// the tokens share are read once; each channel's sum in the order of the kernel above.
constexpr int CONV_TOKENS = 4;

template <int TAPS>
__global__ void __launch_bounds__(128)
causal_conv_silu_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                               int ld, const float* __restrict__ w, const float* __restrict__ bias,
                               const float* __restrict__ state, long state_stride,
                               const int* __restrict__ seq_of_token,
                               const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                               int n_tokens, int channels) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int ROWS = CONV_TOKENS + TAPS - 1;
  const int pieces = channels / 8;
  const int groups = (n_tokens + CONV_TOKENS - 1) / CONV_TOKENS;
  const size_t total = (size_t)groups * pieces;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int tg = (int)(idx / pieces), c = (int)(idx - (size_t)tg * pieces) * 8;
    const int t0 = tg * CONV_TOKENS;
    // the eight channels' weights are 8 x TAPS consecutive floats from a 32-byte boundary
    float wr[8 * TAPS];
#pragma unroll
    for (int i = 0; i < 2 * TAPS; ++i) {
      const float4 q = *reinterpret_cast<const float4*>(w + (size_t)c * TAPS + 4 * i);
      wr[4 * i] = q.x; wr[4 * i + 1] = q.y; wr[4 * i + 2] = q.z; wr[4 * i + 3] = q.w;
    }
    float b8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) b8[e] = bias ? bias[c + e] : 0.f;
    // rows t0 - (TAPS - 1) .. t0 + CONV_TOKENS - 1 of the step, where they exist
    float v[ROWS][8];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int row = t0 - (TAPS - 1) + r;
      if (row >= 0 && row < n_tokens) {
        const uint4 raw = *reinterpret_cast<const uint4*>(x + (size_t)row * ld + c);
        const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in[e]));
          v[r][2 * e] = f.x;
          v[r][2 * e + 1] = f.y;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) v[r][e] = 0.f;
      }
    }
#pragma unroll
    for (int u = 0; u < CONV_TOKENS; ++u) {
      const int t = t0 + u;
      if (t >= n_tokens) break;
      const int s = seq_of_token[t];
      const int local = t - cu_tokens[s];
      float acc[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = b8[e];
      if (local >= TAPS - 1) {
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = fmaf(wr[e * TAPS + j], v[u + j][e], acc[e]);
        }
      } else {
        // the request's first tokens of this step: the inputs before them are in its slot
        const float* st = state + (size_t)slots[s] * state_stride + (size_t)c * (TAPS - 1);
#pragma unroll
        for (int j = 0; j < TAPS; ++j) {
          const int src = local - (TAPS - 1) + j;
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float in = src >= 0 ? v[u + j][e] : st[(size_t)e * (TAPS - 1) + (TAPS - 1) + src];
            acc[e] = fmaf(wr[e * TAPS + j], in, acc[e]);
          }
        }
      }
      uint32_t res[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_bfloat162 o = __floats2bfloat162_rn(acc[2 * e] / (1.f + expf(-acc[2 * e])),
                                                       acc[2 * e + 1] / (1.f + expf(-acc[2 * e + 1])));
        res[e] = *reinterpret_cast<const uint32_t*>(&o);
      }
      *reinterpret_cast<uint4*>(out + (size_t)t * channels + c) = make_uint4(res[0], res[1], res[2], res[3]);
    }
  }
}

template <typename T>
__global__ void causal_conv_state_kernel(float* __restrict__ state, long state_stride,
                                         const T* __restrict__ x, int ld,
                                         const int* __restrict__ cu_tokens,
                                         const int* __restrict__ slots, int n_seqs, int channels,
                                         int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int keep = taps - 1;
  const size_t total = (size_t)n_seqs * channels;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const int s = (int)(idx / channels), c = (int)(idx - (size_t)s * channels);
    const int t0 = cu_tokens[s], n = cu_tokens[s + 1] - t0;
    float* st = state + (size_t)slots[s] * state_stride + (size_t)c * keep;
    // ascending j reads old entries at j + n >= j only: in place is safe
    for (int j = 0; j < keep; ++j) {
      const int src = n - keep + j;
      st[j] = src >= 0 ? to_float(x[(size_t)(t0 + src) * ld + c]) : st[j + n];
    }
  }
}

HB_EXPORT int hb_causal_conv_silu(void* out, const void* x, int ld, const float* w, const float* bias,
                                  float* state,
                                  long state_stride, const int* seq_of_token, const int* cu_tokens,
                                  const int* slots, int n_tokens, int n_seqs, int channels, int taps,
                                  int act_dt, cudaStream_t stream) {
  if (n_tokens <= 0 || channels <= 0) return HB_OK;
  if (taps < 1 || ld < channels) return HB_BAD_ARGUMENT;
  const size_t total = (size_t)n_tokens * channels;
  // steps of few tokens keep a thread a (token, channel): more threads, shorter chains of loads
  if (act_dt == HB_BF16 && n_tokens >= 64 && channels % 8 == 0 && ld % 8 == 0 && taps >= 2 && taps <= 4 &&
      ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) & 15) == 0) {
    size_t vblocks = ((size_t)((n_tokens + CONV_TOKENS - 1) / CONV_TOKENS) * (channels / 8) + 127) / 128;
    if (vblocks > 148 * 32) vblocks = 148 * 32;
#define HB_CONV8(TP)                                                                                          \
    hb_launch(causal_conv_silu_bf16x8_kernel<TP>, dim3((unsigned)vblocks), dim3(128), 0, stream,              \
              (__nv_bfloat16*)out, (const __nv_bfloat16*)x, ld, w, bias, (const float*)state, state_stride,   \
              seq_of_token, cu_tokens, slots, n_tokens, channels)
    if (taps == 2) HB_CONV8(2);
    else if (taps == 3) HB_CONV8(3);
    else HB_CONV8(4);
#undef HB_CONV8
  } else {
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    HB_DISPATCH_DTYPE(act_dt, TA,
      hb_launch(causal_conv_silu_kernel<TA>, dim3((unsigned)blocks), dim3(256), 0, stream, (TA*)out,
                (const TA*)x, ld, w, bias, (const float*)state, state_stride, seq_of_token, cu_tokens, slots,
                n_tokens, channels, taps));
  }
  if (taps > 1) {
    const size_t total2 = (size_t)n_seqs * channels;
    size_t blocks2 = (total2 + 255) / 256;
    if (blocks2 > 148 * 16) blocks2 = 148 * 16;
    HB_DISPATCH_DTYPE(act_dt, TA,
      hb_launch(causal_conv_state_kernel<TA>, dim3((unsigned)blocks2), dim3(256), 0, stream, state,
                state_stride, (const TA*)x, ld, cu_tokens, slots, n_seqs, channels, taps));
  }
  return hb_check_launch();
}

// ---------------------------------------------------------------- the recurrence
// Two kernels.  `delta_prepare` is parallel over (token, head): unit-norm k and q (q also
// times dk^-1/2), the decays g = exp(-exp(A_log) softplus(a + dt_bias)) and the write strength
// beta = sigmoid(b), all float32, left as kqg [T, heads, 3, dkp] (dkp = dk rounded up to 4;
// the padding holds k = q = 0, g = 1) and (beta, k . q) [T, heads, 2].  `delta_rule` then walks each
// request's tokens in order: a block owns 64 columns of one head's S, a quad of threads one
// column in registers (a quarter of its dk rows each); the staged rows of 16 tokens arrive in
// shared memory by 16-byte cp.async one chunk ahead, the values of the next chunk wait in
// registers, and the two sums over dk run as four partial sums a thread and two shuffles
// (their order depends on dk alone, not on the step or the batch).
constexpr int DR_CHUNK = 16;        // tokens staged in shared memory at a time
constexpr int DR_COLS = 64;         // columns of S (threads) a block owns

__device__ __forceinline__ void dr_cp_async16(void* smem, const void* gmem) {
  const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}

// qkv [T, qkv_ld]: q at q_off + kh * dk, k at k_off + kh * dk (after convolution and silu).
// beta_raw [T, beta_ld] at column h (before the sigmoid), a_raw [T, a_ld] at column h * dk
// (before dt_bias and softplus).
template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(float* __restrict__ kqg, float* __restrict__ beta, const T* __restrict__ qkv,
                     int qkv_ld, int q_off, int k_off, const T* __restrict__ beta_raw, int beta_ld,
                     const T* __restrict__ a_raw, int a_ld, const float* __restrict__ a_log,
                     const float* __restrict__ dt_bias, int n_rows, int heads, int kv_heads, int dk,
                     int dkp) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int t = row / heads, h = row - t * heads;
  const int kh = h / (heads / kv_heads);
  const T* kr = qkv + (size_t)t * qkv_ld + k_off + (size_t)kh * dk;
  const T* qr = qkv + (size_t)t * qkv_ld + q_off + (size_t)kh * dk;
  float kk = 0.f, qq = 0.f;
  for (int i = lane; i < dk; i += 32) {
    const float kv = to_float(kr[i]), qv = to_float(qr[i]);
    kk += kv * kv;
    qq += qv * qv;
  }
  const float kn = rsqrtf(warp_sum(kk) + 1e-6f);
  const float qn = rsqrtf(warp_sum(qq) + 1e-6f) * rsqrtf((float)dk);
  const float rate = expf(a_log[h]);
  float* dst = kqg + (size_t)row * 3 * dkp;
  for (int i = lane; i < dkp; i += 32) {
    float kv = 0.f, qv = 0.f, gv = 1.f;
    if (i < dk) {
      kv = to_float(kr[i]) * kn;
      qv = to_float(qr[i]) * qn;
      const float a = to_float(a_raw[(size_t)t * a_ld + (size_t)h * dk + i]) + dt_bias[(size_t)h * dk + i];
      const float sp = a > 20.f ? a : log1pf(expf(a));
      gv = expf(-rate * sp);
    }
    dst[i] = kv;
    dst[dkp + i] = qv;
    dst[2 * dkp + i] = gv;
  }
  // k . q of the unit vectors: the scan reads o = (g (.) S)^T q + u (k . q) off ONE pass over S
  float kq = 0.f;
  for (int i = lane; i < dk; i += 32) kq = fmaf(to_float(kr[i]), to_float(qr[i]), kq);
  kq = warp_sum(kq) * kn * qn;
  if (lane == 0) {
    beta[2 * row] = 1.f / (1.f + expf(-to_float(beta_raw[(size_t)t * beta_ld + h])));
    beta[2 * row + 1] = kq;
  }
}

// v at qkv[t, v_off + h * dv + col].  S of a slot at state + slot * state_stride,
// [heads, dk, dv].  o [T, heads * dv] float32.  A column of S is held by the four threads of
// a quad: thread `part` keeps the rows 16 m + 4 part .. + 3 (the float4 groups m * 4 + part),
// and the two sums over dk are finished with two shuffles.
template <typename T, int DK>
__global__ void __launch_bounds__(DR_COLS * 4)
delta_rule_kernel(float* __restrict__ o, const float* __restrict__ kqg, const float* __restrict__ beta,
                  const T* __restrict__ qkv, int qkv_ld, int v_off, float* __restrict__ state,
                  long state_stride, const int* __restrict__ cu_tokens, const int* __restrict__ slots,
                  int heads, int dk, int dkp, int dv) {
  // Neither launched early nor releasing the next kernel early: a long prompt of one request
  // is a few blocks that run for a millisecond.  Launched while the kernel before still holds
  // the SMs they land two to an SM wherever room is, and share its issue slots for all that
  // time (2,048 tokens of one request: 2.54 ms against 1.10 ms on idle SMs); the blocks of a
  // dependent released at the start would wait beside them as long.
  pdl_wait();
  extern __shared__ __align__(16) float dr_sm[];
  constexpr int THREADS = DR_COLS * 4, G = DK / 16;   // float4 groups a thread holds
  const int row_f = 3 * dkp;                        // staged floats a token
  float* stage_buf = dr_sm;                         // [2][CHUNK][3 dkp]
  float* bs = dr_sm + 2 * DR_CHUNK * row_f;         // [2][CHUNK][2]: beta, k . q
  float* vs = bs + 4 * DR_CHUNK;                    // [2][CHUNK][COLS]
  const int s = blockIdx.x, h = blockIdx.y;
  const int part = threadIdx.x & 3, lcol = threadIdx.x >> 2;
  const int col = blockIdx.z * DR_COLS + lcol;
  const bool live = col < dv;
  const int t0 = cu_tokens[s], n = cu_tokens[s + 1] - t0;
  float* S_g = state + (size_t)slots[s] * state_stride + (size_t)h * dk * dv;
  const T* v_col = qkv + v_off + (size_t)h * dv + (live ? col : 0);

  float S[G][4];
#pragma unroll
  for (int m = 0; m < G; ++m)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int i = 16 * m + 4 * part + e;
      S[m][e] = (live && i < dk) ? S_g[(size_t)i * dv + col] : 0.f;
    }

  auto stage = [&](int c0, int b) {
    const int nc = min(DR_CHUNK, n - c0);
    const int vecs = row_f / 4;
    float* dst = stage_buf + (size_t)b * DR_CHUNK * row_f;
    for (int idx = threadIdx.x; idx < nc * vecs; idx += THREADS) {
      const int j = idx / vecs, v = idx - j * vecs;
      dr_cp_async16(dst + j * row_f + v * 4, kqg + ((size_t)(t0 + c0 + j) * heads + h) * row_f + v * 4);
    }
    for (int j = threadIdx.x; j < 2 * nc; j += THREADS)
      bs[2 * b * DR_CHUNK + j] = beta[2 * ((size_t)(t0 + c0 + (j >> 1)) * heads + h) + (j & 1)];
  };
  // the quad's thread `part` fetches the values of tokens part, part + 4, ... of a chunk
  float v_next[DR_CHUNK / 4];
  auto fetch_v = [&](int c0) {
#pragma unroll
    for (int jj = 0; jj < DR_CHUNK / 4; ++jj) {
      const int j = 4 * jj + part;
      v_next[jj] = (c0 + j < n) ? to_float(v_col[(size_t)(t0 + c0 + j) * qkv_ld]) : 0.f;
    }
  };

  if (n > 0) {
    stage(0, 0);
    fetch_v(0);
  }
  asm volatile("cp.async.commit_group;\n" ::);
  int b = 0;
  for (int c0 = 0; c0 < n; c0 += DR_CHUNK) {
    const int nc = min(DR_CHUNK, n - c0);
    asm volatile("cp.async.wait_group 0;\n" ::);
#pragma unroll
    for (int jj = 0; jj < DR_CHUNK / 4; ++jj) vs[(b * DR_CHUNK + 4 * jj + part) * DR_COLS + lcol] = v_next[jj];
    __syncthreads();
    if (c0 + DR_CHUNK < n) {
      stage(c0 + DR_CHUNK, b ^ 1);
      fetch_v(c0 + DR_CHUNK);
    }
    asm volatile("cp.async.commit_group;\n" ::);
    const float* rows = stage_buf + (size_t)b * DR_CHUNK * row_f;
#pragma unroll 2
    for (int j = 0; j < nc; ++j) {
      const float4* k4 = reinterpret_cast<const float4*>(rows + j * row_f) + part;
      const float4* q4 = reinterpret_cast<const float4*>(rows + j * row_f + dkp) + part;
      const float4* g4 = reinterpret_cast<const float4*>(rows + j * row_f + 2 * dkp) + part;
      // one pass: S <- g (.) S with the sums S^T k and S^T q; then u, the read-out
      // o = S^T q + u (k . q) (what S^T q is after the write), and the write S += k u, which
      // nothing waits for until the next token's pass
      float d0 = 0.f, d1 = 0.f, e0 = 0.f, e1 = 0.f;
      float4 kk[G];
#pragma unroll
      for (int m = 0; m < G; ++m)
        if (16 * m + 4 * part < dkp) {
          const float4 g = g4[4 * m], k = k4[4 * m], q = q4[4 * m];
          kk[m] = k;
          S[m][0] *= g.x; d0 = fmaf(S[m][0], k.x, d0); e0 = fmaf(S[m][0], q.x, e0);
          S[m][1] *= g.y; d1 = fmaf(S[m][1], k.y, d1); e1 = fmaf(S[m][1], q.y, e1);
          S[m][2] *= g.z; d0 = fmaf(S[m][2], k.z, d0); e0 = fmaf(S[m][2], q.z, e0);
          S[m][3] *= g.w; d1 = fmaf(S[m][3], k.w, d1); e1 = fmaf(S[m][3], q.w, e1);
        }
      float dot = d0 + d1, rd = e0 + e1;
      dot += __shfl_xor_sync(0xffffffffu, dot, 1);
      rd += __shfl_xor_sync(0xffffffffu, rd, 1);
      dot += __shfl_xor_sync(0xffffffffu, dot, 2);
      rd += __shfl_xor_sync(0xffffffffu, rd, 2);
      const float u = bs[2 * (b * DR_CHUNK + j)] * (vs[(b * DR_CHUNK + j) * DR_COLS + lcol] - dot);
      const float out = fmaf(u, bs[2 * (b * DR_CHUNK + j) + 1], rd);
#pragma unroll
      for (int m = 0; m < G; ++m)
        if (16 * m + 4 * part < dkp) {
          S[m][0] = fmaf(kk[m].x, u, S[m][0]);
          S[m][1] = fmaf(kk[m].y, u, S[m][1]);
          S[m][2] = fmaf(kk[m].z, u, S[m][2]);
          S[m][3] = fmaf(kk[m].w, u, S[m][3]);
        }
      if (live && part == 0) o[(size_t)(t0 + c0 + j) * heads * dv + (size_t)h * dv + col] = out;
    }
    b ^= 1;
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  if (live) {
#pragma unroll
    for (int m = 0; m < G; ++m)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 16 * m + 4 * part + e;
        if (i < dk) S_g[(size_t)i * dv + col] = S[m][e];
      }
  }
}

// scratch: n_tokens * heads * (3 * dkp + 2) floats, dkp = dk rounded up to a multiple of 4
HB_EXPORT int hb_delta_rule(float* o, float* scratch, const void* qkv, int qkv_ld, int q_off, int k_off,
                            int v_off, const void* beta_raw, int beta_ld, const void* a_raw, int a_ld,
                            const float* a_log, const float* dt_bias, float* state,
                            long state_stride, const int* cu_tokens, const int* slots, int n_tokens,
                            int n_seqs, int heads, int kv_heads, int dk, int dv, int act_dt,
                            cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return HB_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dk <= 0 || dk > 256 || dv <= 0 ||
      heads > 65535 || scratch == nullptr)
    return HB_BAD_ARGUMENT;
  const int dkp = (dk + 3) / 4 * 4;
  float* kqg = scratch;
  float* beta = scratch + (size_t)n_tokens * heads * 3 * dkp;
  const int n_rows = n_tokens * heads;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(delta_prepare_kernel<TA>, dim3((n_rows + 3) / 4), dim3(128), 0, stream, kqg, beta,
              (const TA*)qkv, qkv_ld, q_off, k_off, (const TA*)beta_raw, beta_ld, (const TA*)a_raw, a_ld,
              a_log, dt_bias, n_rows, heads, kv_heads, dk, dkp));
  dim3 grid(n_seqs, heads, (dv + DR_COLS - 1) / DR_COLS);
  const size_t smem = ((size_t)2 * DR_CHUNK * 3 * dkp + 4 * DR_CHUNK + 2 * DR_CHUNK * DR_COLS) * sizeof(float);
#define HB_DR_LAUNCH(DKMAX)                                                                       \
  HB_DISPATCH_DTYPE(act_dt, TA,                                                                   \
    if (smem > 48 * 1024)                                                                         \
      cudaFuncSetAttribute(delta_rule_kernel<TA, DKMAX>,                                          \
                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);               \
    delta_rule_kernel<TA, DKMAX><<<grid, dim3(DR_COLS * 4), smem, stream>>>(                      \
        o, (const float*)kqg, (const float*)beta, (const TA*)qkv, qkv_ld, v_off, state,           \
        state_stride, cu_tokens, slots, heads, dk, dkp, dv))
  if (dk <= 16) HB_DR_LAUNCH(16);
  else if (dk <= 32) HB_DR_LAUNCH(32);
  else if (dk <= 64) HB_DR_LAUNCH(64);
  else if (dk <= 128) HB_DR_LAUNCH(128);
  else HB_DR_LAUNCH(256);
#undef HB_DR_LAUNCH
  return hb_check_launch();
}

// ---------------------------------------------------------------- output norm and gate
// out[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * weight * sigmoid(gate[t, h, :]);
// one warp per (token, head); the weight (dv values) is shared by the heads.
template <typename T>
__global__ void gated_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ o,
                                     const T* __restrict__ gate, int gate_ld,
                                     const float* __restrict__ weight, int n_rows, int heads, int dv,
                                     float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const int t = row / heads, h = row - t * heads;
  const float* orow = o + (size_t)row * dv;
  const T* grow = gate + (size_t)t * gate_ld + (size_t)h * dv;
  float ss = 0.f;
  for (int d = lane; d < dv; d += 32) ss += orow[d] * orow[d];
  const float rstd = rsqrtf(warp_sum(ss) / (float)dv + eps);
  T* dst = out + (size_t)row * dv;
  for (int d = lane; d < dv; d += 32) {
    const float gt = 1.f / (1.f + expf(-to_float(grow[d])));
    dst[d] = from_float<T>(orow[d] * rstd * weight[d] * gt);
  }
}

HB_EXPORT int hb_gated_rmsnorm(void* out, const float* o, const void* gate, int gate_ld,
                               const float* weight, int T, int heads, int dv, float eps, int act_dt,
                               cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (heads <= 0 || dv <= 0 || gate_ld < heads * dv) return HB_BAD_ARGUMENT;
  const int n_rows = T * heads;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(gated_rmsnorm_kernel<TA>, dim3((n_rows + 3) / 4), dim3(128), 0, stream, (TA*)out, o,
              (const TA*)gate, gate_ld, weight, n_rows, heads, dv, eps));
  return hb_check_launch();
}
