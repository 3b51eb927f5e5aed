// What an attention kernel may be asked for beyond scaled dot products, a causal mask and a
// window; everything off in a zeroed struct.
//   slopes  float [heads]: score - slopes[h] * (query position - key position)
//   sink    the softmax has a key of score 0 that carries no value: the weights are
//           exp(s_j) / (1 + sum_j exp(s_j))
//   gate    [tokens, >= heads], rows gate_stride elements apart: head h's output at token t
//           is multiplied by sigmoid(gate[t, h]); with gate_wide the rows hold a gate per
//           output VALUE, gate[t, h * value size + d]
//   bias_table  float [bias_rows, heads]: score + bias_table[min(distance, bias_rows - 1), h]
//   sink_values float [heads]: the sink's score is sink_values[h] instead of 0
//   keep_first  with a window: the request's first keep_first keys stay visible
#pragma once
#include "common.cuh"

struct AttnOptions {
  const float* slopes;
  const __nv_bfloat16* gate;
  int gate_stride;
  int sink;
  const float* bias_table;
  int bias_rows;
  const float* sink_values;
  int keep_first;
  int gate_wide;
};

// One output value from an accumulator `acc` and the row's maximum M (log2 domain) and sum L,
// both relative to M: the sink joins the sum as exp2(0 - M'), M' = max(M, 0); then the gate.
// With no sink and a factor of 1 this is acc / L, bit for bit.
// `sink_log2`: the sink's score in the log2 domain (attn_sink_log2; 0 unless given).
__device__ __forceinline__ float attn_finish(float acc, float M, float L, int sink, float gate_factor,
                                             float sink_log2 = 0.f) {
  if (sink) {
    const float Mn = fmaxf(M, sink_log2);
    const float f = exp2f(M - Mn);
    acc *= f;
    L = L * f + exp2f(sink_log2 - Mn);
  }
  return acc / L * gate_factor;
}

__device__ __forceinline__ float attn_sink_log2(const AttnOptions& opt, int head) {
  return opt.sink_values != nullptr ? opt.sink_values[head] * 1.4426950408889634f : 0.f;
}

// The gate of head `head` at `token`; with gate_wide the gate of its value d of vd.
__device__ __forceinline__ float attn_gate_factor(const AttnOptions& opt, size_t token, int head,
                                                  int d = 0, int vd = 0) {
  if (opt.gate == nullptr) return 1.f;
  const size_t col = opt.gate_wide ? (size_t)head * vd + d : (size_t)head;
  const float g = __bfloat162float(opt.gate[token * (size_t)opt.gate_stride + col]);
  return 1.f / (1.f + __expf(-g));
}

// The bias of a score from the table by distance, in the log2 domain.
__device__ __forceinline__ float attn_table_bias_log2(const AttnOptions& opt, int distance, int head, int nh) {
  const int row = distance < opt.bias_rows ? (distance < 0 ? 0 : distance) : opt.bias_rows - 1;
  return opt.bias_table[(size_t)row * nh + head] * 1.4426950408889634f;
}

// What a decode kernel that takes the step's q | k | v rows straight from the projection does
// to them on the way in, beside (or instead of) a rotation: q and k heads divided by their
// root mean square (eps inside the root) and multiplied by a weight per channel (wq, wk: float
// [head_dim], one for all heads; null: no norm), the query also by
// 1 + coef * ln(floor((position + 1) / every) + 1) (every 0: no such factor).
struct QkPrepare {
  const float* wq;
  const float* wk;
  float eps;
  float coef;
  int every;
};
