// Routed feed-forward: every token runs `top` of `experts` small gated feed-forward layers.
//
//   z = W_router h (float32), s = sigmoid(z); the `top` experts with the largest s are
//   chosen (compared by z, which orders them as s does without saturating; the lower index
//   on a tie); an expert's weight is its s, not renormalised, and
//   multiplies the expert's INPUT:  out = sum over chosen e of expert_e(s_e * h).
//
// `moe_topk` picks experts and weights.  `moe_expert_rows` runs one (token, choice) pair per
// block, streaming that expert's rows (steps of few tokens, where every expert's weights
// are read about once); `moe_combine` adds a token's choices in the order of the choice.
// The gate is the clamped form of `glu_value` in elementwise.cu:
// g' = min(g, limit), u' = clamp(u, -limit, limit), y = g' sigmoid(1.702 g') (u' + 1).
//
// The same kernels serve a second form, chosen by arguments: s = softmax(z) over all router
// outputs; the choice goes by s + correction (a vector the checkpoint brings) while the weight
// stays s; the weight multiplies the expert's OUTPUT; the gate is silu; router outputs from
// `n_real` on stand for experts without tensors that return their input; and a tensor
// `base` (an expert every token runs) is added to the sum.
#include "common.cuh"

constexpr int MOE_MAX_TOP = 16;

// four consecutive values as floats (float32: one 16-byte access; bfloat16: one of 8 bytes)
template <typename T>
__device__ __forceinline__ void moe_load4(const T* p, float (&f)[4]) {
  if constexpr (sizeof(T) == 4) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    f[0] = x.x; f[1] = x.y; f[2] = x.z; f[3] = x.w;
  } else {
    const uint2 x = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
    f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
  }
}
template <typename T>
__device__ __forceinline__ void moe_store4(T* p, const float (&f)[4]) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
  } else {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    uint2 x;
    x.x = *reinterpret_cast<uint32_t*>(&a);
    x.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = x;
  }
}

// MOE_TOP_SOFTMAX: the choice goes by the logits themselves and the weights are a softmax over
// the CHOSEN logits alone.  `bias` (a vector the checkpoint brings) is added to the logits
// before anything else, whatever the kind.
enum { MOE_SIGMOID = 0, MOE_SOFTMAX = 1, MOE_TOP_SOFTMAX = 2 };
// the codes of the gated activations; MOE_ACT_RELU2: an expert WITHOUT a gate,
// down(relu(up x)^2), whose first matrix has ff rows instead of 2 ff
enum { MOE_GATE_SILU = 0, MOE_GATE_CLAMPED_SWISH = 2, MOE_ACT_RELU2 = 3 };

__global__ void moe_topk_kernel(int* __restrict__ ids, float* __restrict__ weights,
                                const float* __restrict__ logits_in,
                                const float* __restrict__ correction, const float* __restrict__ bias,
                                float* __restrict__ biased, int n_tokens, int experts,
                                int top, int kind, int normalize, float weight_scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= n_tokens) return;
  const float* z = logits_in + (size_t)t * experts;
  if (bias) {                       // the logits with their bias, in the caller's scratch rows
    float* zb = biased + (size_t)t * experts;
    for (int e = 0; e < experts; ++e) zb[e] = z[e] + bias[e];
    z = zb;
  }
  // softmax: the scores need the row's maximum and sum (float32, experts in their order)
  float zmax = 0.f, denom = 1.f;
  if (kind == MOE_SOFTMAX) {
    zmax = -INFINITY;
    for (int e = 0; e < experts; ++e) zmax = fmaxf(zmax, z[e]);
    denom = 0.f;
    for (int e = 0; e < experts; ++e) denom += expf(z[e] - zmax);
  }
  // sigmoid scores without a correction are ordered as z is, which does not saturate
  const bool by_logit = ((kind == MOE_SIGMOID) && (correction == nullptr)) || kind == MOE_TOP_SOFTMAX;
  int chosen[MOE_MAX_TOP];
  float top_logit[MOE_MAX_TOP];
  for (int k = 0; k < top; ++k) {
    float best = 0.f, best_score = 0.f;
    int at = -1;
    for (int e = 0; e < experts; ++e) {
      bool taken = false;
      for (int j = 0; j < k; ++j) taken |= (chosen[j] == e);
      if (taken) continue;
      const float s = (kind == MOE_SOFTMAX) ? expf(z[e] - zmax) / denom
                      : (kind == MOE_TOP_SOFTMAX ? z[e] : 1.f / (1.f + expf(-z[e])));
      const float c = by_logit ? z[e] : s + (correction ? correction[e] : 0.f);
      if (at < 0 || c > best) { best = c; best_score = s; at = e; }   // a NaN never wins: `at` stays valid
    }
    chosen[k] = at;
    top_logit[k] = best_score;
    ids[(size_t)t * top + k] = at;
    weights[(size_t)t * top + k] = best_score;
  }
  if (kind == MOE_TOP_SOFTMAX) {    // the first pick holds the largest logit
    float sum = 0.f;
    for (int k = 0; k < top; ++k) { top_logit[k] = expf(top_logit[k] - top_logit[0]); sum += top_logit[k]; }
    for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] = top_logit[k] / sum * weight_scale;
  } else if (normalize || weight_scale != 1.f) {      // the chosen scores over their sum, in the picks' order
    float sum = 0.f;
    for (int k = 0; k < top; ++k) sum += top_logit[k];
    const float f = normalize ? weight_scale / (sum + 1e-20f) : weight_scale;
    for (int k = 0; k < top; ++k) weights[(size_t)t * top + k] = top_logit[k] * f;
  }
}

// The same choice with one warp a token, for up to 32 * MOE_PER_LANE router outputs: lane l
// holds the scores of outputs l, l + 32, ... in registers; maximum and sum of the softmax and
// every pick are warp reductions (a pick: the largest choice value, the lower index on a tie).
// The sums run over the lanes' partial sums in the order of the shuffle tree, whatever the
// batch: a token's weights depend on its own logits alone.
//
// `groups` > 1: the outputs form that many equal runs of neighbours; a run scores the largest
// choice value in it, and only the outputs of the `keep` best runs (the lower index among
// equals) can be chosen.  `normalize`: the weights are the chosen scores over their sum
// (+ 1e-20, added up in the picks' order); `weight_scale` multiplies every weight.
constexpr int MOE_PER_LANE = 8;

__global__ void __launch_bounds__(128)
moe_topk_warp_kernel(int* __restrict__ ids, float* __restrict__ weights,
                     const float* __restrict__ logits, const float* __restrict__ correction,
                     const float* __restrict__ bias, int n_tokens, int experts, int top, int kind,
                     int groups, int keep, int normalize, float weight_scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float group_sm[4][32 * MOE_PER_LANE];     // a warp's choice values, then its runs' scores
  __shared__ unsigned char kept_sm[4][32 * MOE_PER_LANE];
  const int lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (t >= n_tokens) return;
  const float* z = logits + (size_t)t * experts;
  float score[MOE_PER_LANE], choice[MOE_PER_LANE];
  float zmax = -INFINITY;
#pragma unroll
  for (int i = 0; i < MOE_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    score[i] = e < experts ? z[e] + (bias ? bias[e] : 0.f) : -INFINITY;
    zmax = fmaxf(zmax, score[i]);
  }
  const bool by_logit = ((kind == MOE_SIGMOID) && (correction == nullptr)) || kind == MOE_TOP_SOFTMAX;
  if (kind == MOE_SOFTMAX) {
    zmax = warp_max(zmax);
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < MOE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      score[i] = e < experts ? expf(score[i] - zmax) : 0.f;
      part += score[i];
    }
    const float denom = warp_sum(part);
#pragma unroll
    for (int i = 0; i < MOE_PER_LANE; ++i) score[i] = score[i] / denom;
  }
#pragma unroll
  for (int i = 0; i < MOE_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    const float logit = score[i];
    if (kind == MOE_SIGMOID) score[i] = 1.f / (1.f + expf(-logit));     // MOE_TOP_SOFTMAX keeps the logit
    choice[i] = by_logit ? logit : score[i] + ((correction && e < experts) ? correction[e] : 0.f);
  }
  unsigned taken = 0;        // bit i: this lane's i-th output is chosen already (or not eligible)
  if (groups > 1) {
    float* cv = group_sm[threadIdx.x >> 5];
    unsigned char* kept = kept_sm[threadIdx.x >> 5];
    const int per = experts / groups;
#pragma unroll
    for (int i = 0; i < MOE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < experts) cv[e] = choice[i];
    }
    __syncwarp();
    float run[MOE_PER_LANE];             // lane l scores the runs l, l + 32, ...
#pragma unroll
    for (int i = 0; i < MOE_PER_LANE; ++i) {
      const int g = lane + 32 * i;
      float m = -INFINITY;
      if (g < groups)
        for (int e = g * per; e < (g + 1) * per; ++e) m = fmaxf(m, cv[e]);     // a NaN never wins
      run[i] = m;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < MOE_PER_LANE; ++i) {
      const int g = lane + 32 * i;
      if (g < groups) kept[g] = 0;
    }
    unsigned run_taken = 0;
    for (int k = 0; k < keep; ++k) {
      float best = 0.f;
      int at = -1;
#pragma unroll
      for (int i = 0; i < MOE_PER_LANE; ++i) {
        const int g = lane + 32 * i;
        if (g >= groups || (run_taken >> i & 1u)) continue;
        if (at < 0 || run[i] > best) { best = run[i]; at = g; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, at, o);
        if (oa >= 0 && (at < 0 || ob > best || (ob == best && oa < at))) { best = ob; at = oa; }
      }
      if (at >= 0 && (at & 31) == lane) { run_taken |= 1u << (at >> 5); kept[at] = 1; }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < MOE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e < experts && !kept[e / per]) taken |= 1u << i;
    }
  }
  const bool own_weights = kind == MOE_TOP_SOFTMAX || normalize;   // lane k keeps pick k's term
  float first_logit = 0.f, top_sum = 0.f, mine = 0.f;
  for (int k = 0; k < top; ++k) {
    float best = 0.f, best_score = 0.f;
    int at = -1;
#pragma unroll
    for (int i = 0; i < MOE_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (e >= experts || (taken >> i & 1u)) continue;
      if (at < 0 || choice[i] > best || (best != best && choice[i] == choice[i])) {
        best = choice[i]; best_score = score[i]; at = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const float os = __shfl_xor_sync(0xffffffffu, best_score, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      // one order for all lanes, so that they end with the same pick: a number before a NaN,
      // the larger number, and the lower index among equals (and among NaNs)
      const bool on = ob == ob, bn = best == best;
      const bool wins = oa >= 0 && (at < 0 || (on && !bn) ||
                                    (on == bn && ((on && ob > best) || ((!on || ob == best) && oa < at))));
      if (wins) { best = ob; best_score = os; at = oa; }
    }
    if (at >= 0 && (at & 31) == lane) taken |= 1u << (at >> 5);
    if (kind == MOE_TOP_SOFTMAX) {       // picks come largest first; the terms add up in that order
      if (k == 0) first_logit = best_score;
      const float term = expf(best_score - first_logit);
      top_sum += term;
      if (lane == k) mine = term;
      if (lane == 0) ids[(size_t)t * top + k] = at;
    } else if (normalize) {              // the chosen scores add up in the picks' order
      top_sum += best_score;
      if (lane == k) mine = best_score;
      if (lane == 0) ids[(size_t)t * top + k] = at;
    } else if (lane == 0) {
      ids[(size_t)t * top + k] = at;
      weights[(size_t)t * top + k] = best_score * weight_scale;
    }
  }
  if (own_weights && lane < top)
    weights[(size_t)t * top + lane] = mine / (top_sum + (kind == MOE_TOP_SOFTMAX ? 0.f : 1e-20f)) * weight_scale;
}

// `biased`: scratch [n_tokens, experts] for the logits with their bias (rows of more than
// 32 * MOE_PER_LANE router outputs with a bias only)
// `groups`, `keep`: see the warp kernel (rows of up to 32 * MOE_PER_LANE router outputs only)
HB_EXPORT int hb_moe_topk(int* ids, float* weights, const float* logits, const float* correction,
                          const float* bias, float* biased, int n_tokens, int experts, int top, int kind,
                          int groups, int keep, int normalize, float weight_scale, cudaStream_t stream) {
  if (n_tokens <= 0) return HB_OK;
  if (experts <= 0 || top <= 0 || top > experts || top > MOE_MAX_TOP ||
      (kind != MOE_SIGMOID && kind != MOE_SOFTMAX && kind != MOE_TOP_SOFTMAX) || top > 32)
    return HB_BAD_ARGUMENT;
  if (groups < 1 || (groups > 1 && (experts % groups || keep < 1 || keep > groups ||
                                    top > keep * (experts / groups) || experts > 32 * MOE_PER_LANE)) ||
      (normalize && kind == MOE_TOP_SOFTMAX))
    return HB_BAD_ARGUMENT;
  if (experts <= 32 * MOE_PER_LANE) {
    hb_launch(moe_topk_warp_kernel, dim3((n_tokens + 3) / 4), dim3(128), 0, stream, ids, weights,
              logits, correction, bias, n_tokens, experts, top, kind, groups, keep, normalize, weight_scale);
    return hb_check_launch();
  }
  if (bias != nullptr && biased == nullptr) return HB_BAD_ARGUMENT;
  hb_launch(moe_topk_kernel, dim3((n_tokens + 127) / 128), dim3(128), 0, stream, ids, weights,
            logits, correction, bias, biased, n_tokens, experts, top, kind, normalize, weight_scale);
  return hb_check_launch();
}

// w_gate_up [experts, 2 ff, width] (gate rows, then up rows; [experts, ff, width] for experts
// without a gate), w_down [experts, width, ff].
// h [T, width] in the activation dtype.  partial [T * top, width] float32.
template <typename T>
__global__ void __launch_bounds__(256)
moe_expert_rows_kernel(float* __restrict__ partial, const T* __restrict__ h,
                       const T* __restrict__ w_gate_up, const T* __restrict__ w_down,
                       const int* __restrict__ ids, const float* __restrict__ weights, int top,
                       int width, int ff, float limit, int gate_kind, int weight_output, int n_real) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float sm[];
  float* x = sm;                 // [width]
  float* y = sm + width;         // [ff]
  const int pair = blockIdx.x;
  const int e = ids[pair];
  const float w = weights[pair];
  const int t = pair / top;
  const T* hr = h + (size_t)t * width;
  float* dst = partial + (size_t)pair * width;
  if (e >= n_real) {               // an expert without tensors: its output is its input
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = w * to_float(hr[c]);
    return;
  }
  const float w_in = weight_output ? 1.f : w, w_out = weight_output ? w : 1.f;
  // the expert's input, rounded as the activation dtype rounds it
  for (int c = threadIdx.x; c < width; c += blockDim.x)
    x[c] = to_float(from_float<T>(w_in * to_float(hr[c])));
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
  const bool gated = gate_kind != MOE_ACT_RELU2;
  const T* wg = w_gate_up + (size_t)e * (gated ? 2 : 1) * ff * width;
  for (int f = warp; f < ff; f += n_warps) {
    const T* gr = wg + (size_t)f * width;
    if (!gated) {                  // the one matrix of an expert without a gate
      float u = 0.f;
      for (int c = lane; c < width; c += 32) u = fmaf(to_float(gr[c]), x[c], u);
      u = warp_sum(u);
      if (lane == 0) {
        u = fmaxf(to_float(from_float<T>(u)), 0.f);
        y[f] = to_float(from_float<T>(u * u));
      }
      continue;
    }
    const T* ur = wg + (size_t)(ff + f) * width;
    float g = 0.f, u = 0.f;
    for (int c = lane; c < width; c += 32) {
      g = fmaf(to_float(gr[c]), x[c], g);
      u = fmaf(to_float(ur[c]), x[c], u);
    }
    g = warp_sum(g);
    u = warp_sum(u);
    if (lane == 0) {
      g = to_float(from_float<T>(g));
      u = to_float(from_float<T>(u));
      if (gate_kind == MOE_GATE_SILU) {
        y[f] = to_float(from_float<T>(g / (1.f + expf(-g)) * u));
      } else {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        y[f] = to_float(from_float<T>(g / (1.f + expf(-1.702f * g)) * (u + 1.f)));
      }
    }
  }
  __syncthreads();
  const T* wd = w_down + (size_t)e * width * ff;
  for (int c = warp; c < width; c += n_warps) {
    const T* dr = wd + (size_t)c * ff;
    float a = 0.f;
    for (int f = lane; f < ff; f += 32) a = fmaf(to_float(dr[f]), y[f], a);
    a = warp_sum(a);
    if (lane == 0) dst[c] = w_out * a;
  }
}

HB_EXPORT int hb_moe_expert_rows(float* partial, const void* h, const void* w_gate_up,
                                 const void* w_down, const int* ids, const float* weights,
                                 int n_tokens, int top, int width, int ff, float limit,
                                 int gate_kind, int weight_output, int n_real, int act_dt,
                                 cudaStream_t stream) {
  if (n_tokens <= 0) return HB_OK;
  if (top <= 0 || width <= 0 || ff <= 0 || n_real < 0 ||
      (gate_kind != MOE_GATE_SILU && gate_kind != MOE_GATE_CLAMPED_SWISH && gate_kind != MOE_ACT_RELU2))
    return HB_BAD_ARGUMENT;
  const size_t smem = (size_t)(width + ff) * sizeof(float);
  if (smem > 200 * 1024) return HB_BAD_ARGUMENT;
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(moe_expert_rows_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)smem);
    hb_launch(moe_expert_rows_kernel<TA>, dim3(n_tokens * top), dim3(256), smem, stream,
              partial, (const TA*)h, (const TA*)w_gate_up, (const TA*)w_down, ids, weights, top, width,
              ff, limit, gate_kind, weight_output, n_real));
  return hb_check_launch();
}

// out[t, :] = base[t, :] (if given) + sum over k of partial[t * top + k, :], k = 0..top-1 in that order
template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const float* __restrict__ partial,
                                   const T* __restrict__ base, size_t total, int width, int top) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / width;
    const int c = (int)(idx - t * width);
    float a = 0.f;
    for (int k = 0; k < top; ++k) a += partial[(t * top + k) * width + c];
    if (base) a += to_float(base[idx]);
    out[idx] = from_float<T>(a);
  }
}

HB_EXPORT int hb_moe_combine(void* out, const float* partial, const void* base, int n_tokens,
                             int width, int top, int act_dt, cudaStream_t stream) {
  if (n_tokens <= 0) return HB_OK;
  const size_t total = (size_t)n_tokens * width;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(moe_combine_kernel<TA>, dim3((unsigned)blocks), dim3(256), 0, stream, (TA*)out,
              partial, (const TA*)base, total, width, top));
  return hb_check_launch();
}

// ---------------------------------------------------------------- steps of many tokens
// The (token, choice) pairs are put in the order of their experts, so that every expert's
// rows are one contiguous run and the two products of all experts are one grouped matrix
// product each.  `moe_sort`: ends[e] = number of pairs of experts 0..e (the run of expert e
// is [ends[e-1], ends[e])), place[pair] = the pair's row in that order.  One block; the
// order inside a run is whatever the atomics give, which no result depends on: a row's
// product is the same wherever it lies.
__global__ void __launch_bounds__(1024)
moe_sort_kernel(int* __restrict__ ends, int* __restrict__ place, const int* __restrict__ ids,
                int n_pairs, int experts) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int cursor[];          // [experts]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) cursor[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&cursor[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      const int c = cursor[e];
      cursor[e] = run;
      run += c;
      ends[e] = run;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) place[i] = atomicAdd(&cursor[ids[i]], 1);
}

HB_EXPORT int hb_moe_sort(int* ends, int* place, const int* ids, int n_pairs, int experts,
                          cudaStream_t stream) {
  if (n_pairs <= 0) return HB_OK;
  if (experts <= 0 || experts > 8192) return HB_BAD_ARGUMENT;
  hb_launch(moe_sort_kernel, dim3(1), dim3(1024), (size_t)experts * sizeof(int), stream, ends, place,
            ids, n_pairs, experts);
  return hb_check_launch();
}

// rows[place[pair], :] = weight[pair] * h[pair / top, :], rounded to the activation dtype
// (weights null: the row itself)
template <typename T>
__global__ void moe_scatter_rows_kernel(T* __restrict__ rows, const T* __restrict__ h,
                                        const int* __restrict__ place,
                                        const float* __restrict__ weights, int top, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int pair = blockIdx.x;
  const T* src = h + (size_t)(pair / top) * width;
  T* dst = rows + (size_t)place[pair] * width;
  if (weights == nullptr) {
    // a plain copy: 16-byte pieces where rows are made of them
    constexpr int PER = 16 / (int)sizeof(T);
    if (width % PER == 0 && ((uintptr_t)src % 16) == 0 && ((uintptr_t)dst % 16) == 0) {
      for (int c = threadIdx.x; c < width / PER; c += blockDim.x)
        reinterpret_cast<uint4*>(dst)[c] = reinterpret_cast<const uint4*>(src)[c];
      return;
    }
    for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = src[c];
    return;
  }
  const float w = weights[pair];
  for (int c = threadIdx.x; c < width; c += blockDim.x) dst[c] = from_float<T>(w * to_float(src[c]));
}

HB_EXPORT int hb_moe_scatter_rows(void* rows, const void* h, const int* place, const float* weights,
                                  int n_tokens, int top, int width, int act_dt, cudaStream_t stream) {
  if (n_tokens <= 0) return HB_OK;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(moe_scatter_rows_kernel<TA>, dim3(n_tokens * top), dim3(256), 0, stream, (TA*)rows,
              (const TA*)h, place, weights, top, width));
  return hb_check_launch();
}

// out[t, :] = base[t, :] + sum over k = 0..top-1, in that order, of w_k * y_k, where y_k is
// rows[place[t * top + k], :], or h[t, :] itself for a pair whose expert id is n_real or more
// (an expert without tensors); w_k = weights[t * top + k], or 1 with weights null.  base, ids,
// weights and h may be null (then: no base, no such experts, no weights).  float32 sums.
template <typename T>
__global__ void moe_gather_sum_kernel(T* __restrict__ out, const T* __restrict__ rows,
                                      const int* __restrict__ place, const int* __restrict__ ids,
                                      const float* __restrict__ weights, const T* __restrict__ h,
                                      const T* __restrict__ base, int n_real, int top, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  // where every choice's row lies and what it weighs, once; then the columns
  __shared__ const T* src[MOE_MAX_TOP];
  __shared__ float wgt[MOE_MAX_TOP];
  if (threadIdx.x < top) {
    const int pair = t * top + threadIdx.x;
    const bool same = ids != nullptr && ids[pair] >= n_real;
    src[threadIdx.x] = same ? h + (size_t)t * width : rows + (size_t)place[pair] * width;
    wgt[threadIdx.x] = weights ? weights[pair] : 1.f;
  }
  __syncthreads();
  const bool weighted = weights != nullptr;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float a = 0.f;
    for (int k = 0; k < top; ++k) {
      const float y = to_float(src[k][c]);
      a = weighted ? fmaf(wgt[k], y, a) : a + y;
    }
    if (base) a += to_float(base[(size_t)t * width + c]);
    out[(size_t)t * width + c] = from_float<T>(a);
  }
}

// The same with four columns a thread (rows of whole 8- or 16-byte pieces): the loads of all
// choices are on their way before the first sum.
template <typename T>
__global__ void moe_gather_sum_vec_kernel(T* __restrict__ out, const T* __restrict__ rows,
                                          const int* __restrict__ place, const int* __restrict__ ids,
                                          const float* __restrict__ weights, const T* __restrict__ h,
                                          const T* __restrict__ base, int n_real, int top, int width) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  __shared__ const T* src[MOE_MAX_TOP];
  __shared__ float wgt[MOE_MAX_TOP];
  if (threadIdx.x < top) {
    const int pair = t * top + threadIdx.x;
    const bool same = ids != nullptr && ids[pair] >= n_real;
    src[threadIdx.x] = same ? h + (size_t)t * width : rows + (size_t)place[pair] * width;
    wgt[threadIdx.x] = weights ? weights[pair] : 1.f;
  }
  __syncthreads();
  const bool weighted = weights != nullptr;
  for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
    float a[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top; ++k) {
      float y[4];
      moe_load4(src[k] + c, y);
#pragma unroll
      for (int e = 0; e < 4; ++e) a[e] = weighted ? fmaf(wgt[k], y[e], a[e]) : a[e] + y[e];
    }
    if (base) {
      float y[4];
      moe_load4(base + (size_t)t * width + c, y);
#pragma unroll
      for (int e = 0; e < 4; ++e) a[e] += y[e];
    }
    moe_store4(out + (size_t)t * width + c, a);
  }
}

HB_EXPORT int hb_moe_gather_sum(void* out, const void* rows, const int* place, const int* ids,
                                const float* weights, const void* h, const void* base, int n_real,
                                int n_tokens, int top, int width, int act_dt, cudaStream_t stream) {
  if (n_tokens <= 0) return HB_OK;
  if (ids != nullptr && h == nullptr) return HB_BAD_ARGUMENT;
  if (top > MOE_MAX_TOP) return HB_BAD_ARGUMENT;
  const bool vec = width % 8 == 0 && (uintptr_t)out % 16 == 0 && (uintptr_t)rows % 16 == 0 &&
                   (uintptr_t)h % 16 == 0 && (uintptr_t)base % 16 == 0;
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (vec) hb_launch(moe_gather_sum_vec_kernel<TA>, dim3(n_tokens), dim3(256), 0, stream, (TA*)out,
                       (const TA*)rows, place, ids, weights, (const TA*)h, (const TA*)base, n_real, top, width);
    else hb_launch(moe_gather_sum_kernel<TA>, dim3(n_tokens), dim3(256), 0, stream, (TA*)out,
                   (const TA*)rows, place, ids, weights, (const TA*)h, (const TA*)base, n_real, top, width));
  return hb_check_launch();
}
