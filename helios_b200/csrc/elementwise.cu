// Embedding gather, fused residual-add + RMSNorm, rotary encoding fused with the
// write of keys and values into cache pages, SwiGLU gating.
//
// The residual stream is always float32; "act" tensors (GEMM inputs and
// outputs, cache pages) are float32 or bfloat16 by a type code.  Statistics,
// angles and sums are float32 in both modes.
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// out[t, :] (f32) = table[ids[t], :] * scale      python/helios/exec/model.py:486
// (scale: a constant some designs put on the embedded tokens; 1 for none; the product is float32)
template <typename T>
__global__ void embedding_kernel(float* __restrict__ out, const T* __restrict__ table,
                                 const int* __restrict__ ids, int H, int V, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;  // ids are validated on the host
  const T* row = table + (size_t)id * H;
  float* o = out + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] = to_float(row[i]) * scale;
}

// bfloat16 table, rows of whole 16-byte chunks: 8 values per thread and trip
__global__ void embedding_bf16x8_kernel(float* __restrict__ out, const __nv_bfloat16* __restrict__ table,
                                        const int* __restrict__ ids, int H, int V, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = ids[t];
  if (id < 0 || id >= V) id = 0;
  const uint4* row = reinterpret_cast<const uint4*>(table + (size_t)id * H);
  float4* o = reinterpret_cast<float4*>(out + (size_t)t * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) {
    const uint4 x = row[i];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&x);
    o[2 * i] = make_float4(__low2float(p[0]) * scale, __high2float(p[0]) * scale, __low2float(p[1]) * scale,
                           __high2float(p[1]) * scale);
    o[2 * i + 1] = make_float4(__low2float(p[2]) * scale, __high2float(p[2]) * scale, __low2float(p[3]) * scale,
                               __high2float(p[3]) * scale);
  }
}

HB_EXPORT int hb_embedding(float* out, const void* table, const int* ids, int T, int H, int V,
                           int table_dt, float scale, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (table_dt == HB_BF16 && H % 8 == 0 && (uintptr_t)table % 16 == 0 && (uintptr_t)out % 16 == 0) {
    hb_launch(embedding_bf16x8_kernel, dim3(T), dim3(256), 0, stream, out, (const __nv_bfloat16*)table, ids, H, V,
              scale);
    return hb_check_launch();
  }
  HB_DISPATCH_DTYPE(table_dt, TT,
    hb_launch(embedding_kernel<TT>, dim3(T), dim3(256), 0, stream, out, (const TT*)table, ids, H, V, scale));
  return hb_check_launch();
}

// ---------------------------------------------------------------- add + RMSNorm
// residual[r] += delta[r] (if delta); out[i] = residual[r] * rsqrt(mean(residual[r]^2) + eps) * w
// where r = rows ? rows[i] : i.  With `rows` the residual is not written back
// (the final norm runs on the wanted rows only).    python/helios/exec/model.py:109-114
//
// A row is held in registers between the two passes (groups of four values per thread,
// all loads issued before the first use), so a row costs one trip to memory.
template <typename T> struct Vec4 { T v[4]; };

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&f)[4]) {
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
__device__ __forceinline__ void store4(T* p, const float (&f)[4]) {
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

constexpr int NORM_THREADS = 256;
constexpr int NORM_GROUPS = 8;     // groups of 4 values a thread keeps: rows up to 8192 wide

template <typename TA, bool VEC>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_kernel(TA* __restrict__ out, float* __restrict__ residual, const TA* __restrict__ delta,
                   const float* __restrict__ weight, const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * H;
  const TA* d = delta ? delta + (size_t)r * H : nullptr;
  const bool write_back = (rows == nullptr) && (d != nullptr);
  TA* o = out + (size_t)i * H;
  float ss = 0.f;
  if constexpr (VEC) {
    float v[NORM_GROUPS][4];
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) load4(res + c, v[g]);
    }
    if (d) {
#pragma unroll
      for (int g = 0; g < NORM_GROUPS; ++g) {
        const int c = (g * NORM_THREADS + threadIdx.x) * 4;
        if (c < H) {
          float dv[4];
          load4(d + c, dv);
#pragma unroll
          for (int e = 0; e < 4; ++e) v[g][e] += dv[e];
        }
      }
    }
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) {
        if (write_back) store4(res + c, v[g]);
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += v[g][e] * v[g][e];
      }
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) {
        float w[4], y[4];
        load4(weight + c, w);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = v[g][e] * rstd * w[e];
        store4(o + c, y);
      }
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float v = res[c];
      if (d) v += to_float(d[c]);
      if (write_back) res[c] = v;
      ss += v * v;
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float v = res[c];
      if (d && !write_back) v += to_float(d[c]);
      o[c] = from_float<TA>(v * rstd * weight[c]);
    }
  }
}

HB_EXPORT int hb_add_rmsnorm(void* out, float* residual, const void* delta, const float* weight,
                             const int* rows, int n_out, int H, float eps, int act_dt,
                             cudaStream_t stream) {
  if (n_out <= 0) return HB_OK;
  // the register-resident path needs whole groups of four and 16-byte aligned rows
  const bool vec = (H % 4 == 0) && H <= NORM_THREADS * NORM_GROUPS * 4 &&
                   ((uintptr_t)out % 16 == 0) && ((uintptr_t)residual % 16 == 0) &&
                   ((uintptr_t)delta % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                   (act_dt == HB_F32 || H % 8 == 0);
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (vec) hb_launch(add_rmsnorm_kernel<TA, true>, dim3(n_out), dim3(NORM_THREADS), 0, stream, 
        (TA*)out, residual, (const TA*)delta, weight, rows, H, eps);
    else hb_launch(add_rmsnorm_kernel<TA, false>, dim3(n_out), dim3(NORM_THREADS), 0, stream, 
        (TA*)out, residual, (const TA*)delta, weight, rows, H, eps));
  return hb_check_launch();
}

// ---------------------------------------------------------------- add + two RMSNorms of one row
// A block whose mixer and feed-forward each read a norm of their own of the SAME stream:
//   residual[r] += a[r] + b[r]                       (float32; a, b optional: what the block before left)
//   out1[r] = residual[r] * rstd * w1,   out2[r] = residual[r] * rstd * w2      (out2 / w2 optional)
// with one rstd = rsqrt(mean(residual[r]^2) + eps) for both.  The row stays in registers (whole
// groups of four) or is read again (other widths).
template <typename TA, bool VEC>
__global__ void __launch_bounds__(NORM_THREADS)
add_rmsnorm_pair_kernel(TA* __restrict__ out1, TA* __restrict__ out2, float* __restrict__ residual,
                        const TA* __restrict__ a, const TA* __restrict__ b,
                        const float* __restrict__ w1, const float* __restrict__ w2, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int r = blockIdx.x;
  float* res = residual + (size_t)r * H;
  const TA* ar = a ? a + (size_t)r * H : nullptr;
  const TA* br = b ? b + (size_t)r * H : nullptr;
  const bool write_back = ar != nullptr || br != nullptr;
  TA* o1 = out1 + (size_t)r * H;
  TA* o2 = out2 ? out2 + (size_t)r * H : nullptr;
  float ss = 0.f;
  if constexpr (VEC) {
    float v[NORM_GROUPS][4];
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) load4(res + c, v[g]);
    }
    if (write_back) {
#pragma unroll
      for (int g = 0; g < NORM_GROUPS; ++g) {
        const int c = (g * NORM_THREADS + threadIdx.x) * 4;
        if (c < H) {
          float add[4] = {0.f, 0.f, 0.f, 0.f}, x[4];
          if (ar) { load4(ar + c, x);
#pragma unroll
            for (int e = 0; e < 4; ++e) add[e] = x[e]; }
          if (br) { load4(br + c, x);
#pragma unroll
            for (int e = 0; e < 4; ++e) add[e] += x[e]; }
#pragma unroll
          for (int e = 0; e < 4; ++e) v[g][e] += add[e];
          store4(res + c, v[g]);
        }
      }
    }
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) {
#pragma unroll
        for (int e = 0; e < 4; ++e) ss = fmaf(v[g][e], v[g][e], ss);
      }
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) {
        float w[4], y[4];
        load4(w1 + c, w);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = v[g][e] * rstd * w[e];
        store4(o1 + c, y);
        if (o2) {
          load4(w2 + c, w);
#pragma unroll
          for (int e = 0; e < 4; ++e) y[e] = v[g][e] * rstd * w[e];
          store4(o2 + c, y);
        }
      }
    }
  } else {
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      float v = res[c];
      if (write_back) {
        float add = ar ? to_float(ar[c]) : 0.f;
        if (br) add += to_float(br[c]);
        v += add;
        res[c] = v;
      }
      ss = fmaf(v, v, ss);
    }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
    for (int c = threadIdx.x; c < H; c += blockDim.x) {
      const float v = res[c];          // this thread's own write, or the row as it was
      o1[c] = from_float<TA>(v * rstd * w1[c]);
      if (o2) o2[c] = from_float<TA>(v * rstd * w2[c]);
    }
  }
}

HB_EXPORT int hb_add_rmsnorm_pair(void* out1, void* out2, float* residual, const void* a, const void* b,
                                  const float* w1, const float* w2, int n_rows, int H, float eps,
                                  int act_dt, cudaStream_t stream) {
  if (n_rows <= 0) return HB_OK;
  if (H <= 0 || out1 == nullptr || w1 == nullptr || ((out2 == nullptr) != (w2 == nullptr)))
    return HB_BAD_ARGUMENT;
  const bool vec = (H % 4 == 0) && H <= NORM_THREADS * NORM_GROUPS * 4 && ((uintptr_t)out1 % 16 == 0) &&
                   ((uintptr_t)out2 % 16 == 0) && ((uintptr_t)residual % 16 == 0) &&
                   ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) && ((uintptr_t)w1 % 16 == 0) &&
                   ((uintptr_t)w2 % 16 == 0) && (act_dt == HB_F32 || H % 8 == 0);
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (vec) hb_launch(add_rmsnorm_pair_kernel<TA, true>, dim3(n_rows), dim3(NORM_THREADS), 0, stream,
                       (TA*)out1, (TA*)out2, residual, (const TA*)a, (const TA*)b, w1, w2, H, eps);
    else hb_launch(add_rmsnorm_pair_kernel<TA, false>, dim3(n_rows), dim3(NORM_THREADS), 0, stream,
                   (TA*)out1, (TA*)out2, residual, (const TA*)a, (const TA*)b, w1, w2, H, eps));
  return hb_check_launch();
}

// ---------------------------------------------------------------- plain RMSNorm of act rows
template <typename T>
__global__ void rmsnorm_kernel(T* __restrict__ out, const T* __restrict__ x,
                               const float* __restrict__ weight, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const T* xr = x + (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) { float v = to_float(xr[c]); ss += v * v; }
  const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
  T* o = out + (size_t)blockIdx.x * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    o[c] = from_float<T>(to_float(xr[c]) * rstd * weight[c]);
}

HB_EXPORT int hb_rmsnorm(void* out, const void* x, const float* weight, int n, int H, float eps,
                         int act_dt, cudaStream_t stream) {
  if (n <= 0) return HB_OK;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(rmsnorm_kernel<TA>, dim3(n), dim3(256), 0, stream, (TA*)out, (const TA*)x, weight, H, eps));
  return hb_check_launch();
}

// ---------------------------------------------------------------- rotary tables
// cos/sin[t, j] of angle = position[t] * inv_freq[j], the product and the functions in
// float64, the result rounded to float32 (python/helios/exec/model.py:127-132 builds the
// same table for every position up to max_position_embeddings).
__global__ void rotary_table_kernel(float* __restrict__ cos_out, float* __restrict__ sin_out,
                                    const int* __restrict__ positions,
                                    const double* __restrict__ inv_freq, int T, int half,
                                    double factor) {
  pdl_launch_dependents();
  pdl_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= T * half) return;
  const int t = idx / half, j = idx - t * half;
  double s, c;
  sincos((double)positions[t] * inv_freq[j], &s, &c);
  cos_out[idx] = (float)(c * factor);
  sin_out[idx] = (float)(s * factor);
}

HB_EXPORT int hb_rotary_table(float* cos_out, float* sin_out, const int* positions,
                              const double* inv_freq, int T, int half, double factor,
                              cudaStream_t stream) {
  if (T <= 0 || half <= 0) return HB_OK;
  const int total = T * half;
  hb_launch(rotary_table_kernel, dim3((total + 127) / 128), dim3(128), 0, stream, cos_out, sin_out, positions,
                                                               inv_freq, T, half, factor);
  return hb_check_launch();
}

// ---------------------------------------------------------------- rotary + cache write
// qkv: [T, (nh + 2 nkv) * hd], q heads first, then k heads, then v heads.
// For every token: rotate q and k (rotate-half pairs (j, j + rot/2) by the token's
// cos/sin row, float32; python/helios/exec/model.py:148-153), leave q in place, and
// store the rotated k and the v at the token's place in its pages
// (python/helios/exec/paged_attn.py:74-85): page = block_table[seq, pos / page],
// pages laid out [page, kv head, slot, hd].
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, const float* __restrict__ cos_tab,
                                     const float* __restrict__ sin_tab,
                                     const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token,
                                     const int* __restrict__ block_table, int bt_stride,
                                     T* __restrict__ k_pages, T* __restrict__ v_pages,
                                     int nh, int nkv, int hd, int rot, int page_size,
                                     int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = rot >> 1;
  const float* cs = cos_tab + (size_t)t * half;
  const float* sn = sin_tab + (size_t)t * half;
  T* row = qkv + (size_t)t * (size_t)(nh + 2 * nkv) * hd;
  size_t page_base = 0;
  int slot = 0;
  if (write_cache) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    slot = pos % page_size;
    page_base = (size_t)page * nkv;
  }
  // rotated pairs of q and k heads
  const int n_rot_heads = nh + nkv;
  for (int w = threadIdx.x; w < n_rot_heads * half; w += blockDim.x) {
    const int h = w / half, j = w - h * half;
    T* x = row + (size_t)h * hd;
    const float x1 = to_float(x[j]), x2 = to_float(x[j + half]);
    const float c = cs[j], s = sn[j];
    const T r1 = from_float<T>(x1 * c - x2 * s);
    const T r2 = from_float<T>(x2 * c + x1 * s);
    if (h < nh || !write_cache) {
      x[j] = r1;
      x[j + half] = r2;
    } else {
      T* dst = k_pages + ((page_base + (h - nh)) * page_size + slot) * hd;
      dst[j] = r1;
      dst[j + half] = r2;
    }
  }
  if (!write_cache) return;
  // un-rotated tail of k (rot < hd), and v
  if (rot < hd) {
    const int tail = hd - rot;
    for (int w = threadIdx.x; w < nkv * tail; w += blockDim.x) {
      const int h = w / tail, j = rot + (w - h * tail);
      k_pages[((page_base + h) * page_size + slot) * hd + j] = row[(size_t)(nh + h) * hd + j];
    }
  }
  for (int w = threadIdx.x; w < nkv * hd; w += blockDim.x) {
    const int h = w / hd, j = w - h * hd;
    v_pages[((page_base + h) * page_size + slot) * hd + j] = row[(size_t)(nh + nkv + h) * hd + j];
  }
}

// The same, four rotary pairs (or eight copied values) per thread, for full rotation
// (rot == hd) with hd a multiple of 8: one block of work items per token is
// (nh + nkv) * hd / 8 rotations followed by nkv * hd / 8 copies of v.
template <typename T>
__global__ void rope_kv_write_vec_kernel(T* __restrict__ qkv, const float* __restrict__ cos_tab,
                                         const float* __restrict__ sin_tab,
                                         const int* __restrict__ positions,
                                         const int* __restrict__ seq_of_token,
                                         const int* __restrict__ block_table, int bt_stride,
                                         T* __restrict__ k_pages, T* __restrict__ v_pages,
                                         int nh, int nkv, int hd, int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int item = blockIdx.y * blockDim.x + threadIdx.x;
  const int half = hd >> 1, quads = half >> 2;            // groups of 4 pairs per head
  const int n_rot = (nh + nkv) * quads;
  const int n_copy = write_cache ? nkv * (hd >> 3) : 0;   // groups of 8 values of v
  if (item >= n_rot + n_copy) return;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * (size_t)(nh + 2 * nkv) * hd;
  size_t page_base = 0;
  int slot = 0;
  if (write_cache) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    slot = pos % page_size;
    page_base = (size_t)page * nkv;
  }
  if (item < n_rot) {
    const int h = item / quads, j = (item - h * quads) * 4;
    T* x = row + (size_t)h * hd;
    float x1[4], x2[4], c[4], sn[4], r1[4], r2[4];
    load4(x + j, x1);
    load4(x + j + half, x2);
    load4(cos_tab + (size_t)t * half + j, c);
    load4(sin_tab + (size_t)t * half + j, sn);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // round as the scalar kernel does: each product pair in float32, one rounding to T
      r1[e] = x1[e] * c[e] - x2[e] * sn[e];
      r2[e] = x2[e] * c[e] + x1[e] * sn[e];
    }
    T* dst = x;
    if (h >= nh && write_cache) dst = k_pages + ((page_base + (h - nh)) * page_size + slot) * hd;
    store4(dst + j, r1);
    store4(dst + j + half, r2);
  } else {
    const int w = item - n_rot;
    const int per = hd >> 3;
    const int h = w / per, j = (w - h * per) * 8;
    const T* src = row + (size_t)(nh + nkv + h) * hd + j;
    T* dst = v_pages + ((page_base + h) * page_size + slot) * hd + j;
    float a[4], b[4];
    load4(src, a);
    load4(src + 4, b);
    store4(dst, a);
    store4(dst + 4, b);
  }
}

HB_EXPORT int hb_rope_kv_write(void* qkv, const float* cos_tab, const float* sin_tab,
                               const int* positions, const int* seq_of_token,
                               const int* block_table, int bt_stride, void* k_pages,
                               void* v_pages, int T, int nh, int nkv, int hd, int rot,
                               int page_size, int write_cache, int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (rot < 0 || rot > hd || (rot & 1) || page_size <= 0) return HB_BAD_ARGUMENT;
  const bool vec = rot == hd && hd % 8 == 0 && (uintptr_t)qkv % 16 == 0 &&
                   (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0 &&
                   (uintptr_t)cos_tab % 16 == 0 && (uintptr_t)sin_tab % 16 == 0;
  if (vec) {
    const int items = (nh + nkv) * (hd / 8) + (write_cache ? nkv * (hd / 8) : 0);
    dim3 grid(T, (items + 127) / 128);
    HB_DISPATCH_DTYPE(act_dt, TA,
      hb_launch(rope_kv_write_vec_kernel<TA>, dim3(grid), dim3(128), 0, stream, 
          (TA*)qkv, cos_tab, sin_tab, positions, seq_of_token, block_table, bt_stride,
          (TA*)k_pages, (TA*)v_pages, nh, nkv, hd, page_size, write_cache));
    return hb_check_launch();
  }
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(rope_kv_write_kernel<TA>, dim3(T), dim3(256), 0, stream, 
        (TA*)qkv, cos_tab, sin_tab, positions, seq_of_token, block_table, bt_stride,
        (TA*)k_pages, (TA*)v_pages, nh, nkv, hd, rot, page_size, write_cache));
  return hb_check_launch();
}

// ---------------------------------------------------------------- SwiGLU gate
// out[t, i] = silu(gu[t, i]) * gu[t, I + i]        python/helios/exec/model.py:336-337
template <typename T>
__global__ void silu_mul_kernel(T* __restrict__ out, const T* __restrict__ gu, size_t total, int I) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    const float g = to_float(gu[t * 2 * I + i]);
    const float u = to_float(gu[t * 2 * I + I + i]);
    out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
  }
}

HB_EXPORT int hb_silu_mul(void* out, const void* gate_up, int T, int I, int act_dt,
                          cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(silu_mul_kernel<TA>, dim3((unsigned)blocks), dim3(threads), 0, stream, (TA*)out, (const TA*)gate_up, total, I));
  return hb_check_launch();
}


// ---------------------------------------------------------------- gated activations
// out[t, i] = act(gu[t, i]) * gu[t, I + i] for a feed-forward whose gate and up rows come
// out of one product.  kind 0: silu(g) * u.  kind 1: the tanh form of gelu,
// 0.5 g (1 + tanh(sqrt(2/pi) (g + 0.044715 g^3))) * u.  kind 2: the clamped form
// g' = min(g, limit), u' = clamp(u, -limit, limit), g' sigmoid(1.702 g') (u' + 1).
enum { HB_GLU_SILU = 0, HB_GLU_GELU_TANH = 1, HB_GLU_CLAMPED_SWISH = 2 };

__device__ __forceinline__ float glu_value(float g, float u, int kind, float limit) {
  if (kind == HB_GLU_GELU_TANH) {
    const float z = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.f + tanhf(z)) * u;
  }
  if (kind == HB_GLU_CLAMPED_SWISH) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
  }
  return g / (1.f + expf(-g)) * u;
}

template <typename T>
__global__ void glu_act_kernel(T* __restrict__ out, const T* __restrict__ gu, size_t total, int I,
                               int kind, float limit) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / I;
    const int i = (int)(idx - t * I);
    out[idx] = from_float<T>(glu_value(to_float(gu[t * 2 * I + i]), to_float(gu[t * 2 * I + I + i]),
                                       kind, limit));
  }
}

HB_EXPORT int hb_glu_act(void* out, const void* gate_up, int T, int I, int kind, float limit,
                         int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (kind < 0 || kind > 2) return HB_BAD_ARGUMENT;
  const size_t total = (size_t)T * I;
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(glu_act_kernel<TA>, dim3((unsigned)blocks), dim3(threads), 0, stream, (TA*)out,
              (const TA*)gate_up, total, I, kind, limit));
  return hb_check_launch();
}

// ---------------------------------------------------------------- norm on a sublayer's output
// residual[r, :] += y[r, :] / sqrt(mean(y[r, :]^2) + eps) * weight (float32), for a block
// that norms what a sublayer returns instead of what it reads; `copy` (may be null)
// receives the new residual row in the activation dtype, which is what the next sublayer
// reads.  With y == null only the copy is made.
template <typename TY, typename TC>
__global__ void __launch_bounds__(256)
rmsnorm_add_kernel(float* __restrict__ residual, const TY* __restrict__ y,
                   const float* __restrict__ weight, TC* __restrict__ copy, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  float* res = residual + (size_t)blockIdx.x * H;
  TC* cp = copy ? copy + (size_t)blockIdx.x * H : nullptr;
  if (y == nullptr) {
    for (int c = threadIdx.x; c < H; c += blockDim.x) cp[c] = from_float<TC>(res[c]);
    return;
  }
  const TY* yr = y + (size_t)blockIdx.x * H;
  float ss = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) { const float v = to_float(yr[c]); ss += v * v; }
  const float rstd = rsqrtf(block_sum(ss, scratch) / (float)H + eps);
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float v = res[c] + to_float(yr[c]) * rstd * weight[c];
    res[c] = v;
    if (cp) cp[c] = from_float<TC>(v);
  }
}

HB_EXPORT int hb_rmsnorm_add(float* residual, const void* y, const float* weight, void* copy,
                             int n, int H, float eps, int y_dt, int copy_dt, cudaStream_t stream) {
  if (n <= 0) return HB_OK;
  if (y == nullptr && copy == nullptr) return HB_OK;
  HB_DISPATCH_DTYPE(y_dt, TY,
    HB_DISPATCH_DTYPE(copy_dt, TC,
      hb_launch(rmsnorm_add_kernel<TY, TC>, dim3(n), dim3(256), 0, stream, residual, (const TY*)y,
                weight, (TC*)copy, H, eps)));
  return hb_check_launch();
}

// ---------------------------------------------------------------- layer norm with a pending sum
// A block whose sublayers all read ONE norm of the stream leaves its outputs to be added:
//   residual[r, c] += mult * (sa[c] * a[r, c] + sb[c] * b[r, c])      (float32; a, b, sa, sb optional)
// and the norm that meets the stream next does the add and norms the new row:
//   out[i, c] = (x[c] - mean) * rsqrt(mean((x - mean)^2) + eps) * w[c] + bias[c],   x = residual[r]
// with r = rows ? rows[i] : i.  With `rows` the residual is not written back (the final norm
// runs on the wanted rows only); with `out` null only the add is done.  The row lies in shared
// memory between the passes; mean and variance are two passes over it in float32.
template <typename TA>
__global__ void __launch_bounds__(NORM_THREADS)
add_layernorm_kernel(TA* __restrict__ out, float* __restrict__ residual, const TA* __restrict__ a,
                     const float* __restrict__ sa, const TA* __restrict__ b,
                     const float* __restrict__ sb, float mult, const float* __restrict__ weight,
                     const float* __restrict__ bias, const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_sm[];
  __shared__ float scratch[33];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * H;
  const TA* ar = a ? a + (size_t)r * H : nullptr;
  const TA* br = b ? b + (size_t)r * H : nullptr;
  const bool write_back = (rows == nullptr) && (ar != nullptr || br != nullptr);
  float sum = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float v = res[c];
    float add = 0.f;
    if (ar) add = (sa ? sa[c] : 1.f) * to_float(ar[c]);
    if (br) add = fmaf(sb ? sb[c] : 1.f, to_float(br[c]), add);
    if (ar || br) v = fmaf(mult, add, v);
    if (write_back) res[c] = v;
    row_sm[c] = v;
    sum += v;
  }
  if (out == nullptr) return;
  const float mean = block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    const float d = row_sm[c] - mean;
    sq = fmaf(d, d, sq);
  }
  const float rstd = rsqrtf(block_sum(sq, scratch) / (float)H + eps);
  TA* o = out + (size_t)i * H;
  for (int c = threadIdx.x; c < H; c += blockDim.x) {
    float y = (row_sm[c] - mean) * rstd * weight[c];
    if (bias) y += bias[c];
    o[c] = from_float<TA>(y);
  }
}

// The same with the row in registers (four values a thread and group, rows of whole groups up
// to 8,192 wide): every load is on its way before the first use, so a row costs one trip to
// memory.  The sums run thread by thread, then over the block in its fixed order, as above.
template <typename TA>
__global__ void __launch_bounds__(NORM_THREADS)
add_layernorm_vec_kernel(TA* __restrict__ out, float* __restrict__ residual, const TA* __restrict__ a,
                         const float* __restrict__ sa, const TA* __restrict__ b,
                         const float* __restrict__ sb, float mult, const float* __restrict__ weight,
                         const float* __restrict__ bias, const int* __restrict__ rows, int H, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int i = blockIdx.x;
  const int r = rows ? rows[i] : i;
  float* res = residual + (size_t)r * H;
  const TA* ar = a ? a + (size_t)r * H : nullptr;
  const TA* br = b ? b + (size_t)r * H : nullptr;
  const bool write_back = (rows == nullptr) && (ar != nullptr || br != nullptr);
  float v[NORM_GROUPS][4];
#pragma unroll
  for (int g = 0; g < NORM_GROUPS; ++g) {
    const int c = (g * NORM_THREADS + threadIdx.x) * 4;
    if (c < H) load4(res + c, v[g]);
  }
  if (ar || br) {
#pragma unroll
    for (int g = 0; g < NORM_GROUPS; ++g) {
      const int c = (g * NORM_THREADS + threadIdx.x) * 4;
      if (c < H) {
        float add[4] = {0.f, 0.f, 0.f, 0.f};
        if (ar) {
          float x[4], s4[4] = {1.f, 1.f, 1.f, 1.f};
          load4(ar + c, x);
          if (sa) load4(sa + c, s4);
#pragma unroll
          for (int e = 0; e < 4; ++e) add[e] = s4[e] * x[e];
        }
        if (br) {
          float x[4], s4[4] = {1.f, 1.f, 1.f, 1.f};
          load4(br + c, x);
          if (sb) load4(sb + c, s4);
#pragma unroll
          for (int e = 0; e < 4; ++e) add[e] = fmaf(s4[e], x[e], add[e]);
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) v[g][e] = fmaf(mult, add[e], v[g][e]);
        if (write_back) store4(res + c, v[g]);
      }
    }
  }
  if (out == nullptr) return;
  float sum = 0.f;
#pragma unroll
  for (int g = 0; g < NORM_GROUPS; ++g) {
    const int c = (g * NORM_THREADS + threadIdx.x) * 4;
    if (c < H) sum += (v[g][0] + v[g][1]) + (v[g][2] + v[g][3]);
  }
  const float mean = block_sum(sum, scratch) / (float)H;
  float sq = 0.f;
#pragma unroll
  for (int g = 0; g < NORM_GROUPS; ++g) {
    const int c = (g * NORM_THREADS + threadIdx.x) * 4;
    if (c < H) {
#pragma unroll
      for (int e = 0; e < 4; ++e) { const float d = v[g][e] - mean; sq = fmaf(d, d, sq); }
    }
  }
  const float rstd = rsqrtf(block_sum(sq, scratch) / (float)H + eps);
  TA* o = out + (size_t)i * H;
#pragma unroll
  for (int g = 0; g < NORM_GROUPS; ++g) {
    const int c = (g * NORM_THREADS + threadIdx.x) * 4;
    if (c < H) {
      float w[4], bb[4] = {0.f, 0.f, 0.f, 0.f}, y[4];
      load4(weight + c, w);
      if (bias) load4(bias + c, bb);
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = (v[g][e] - mean) * rstd * w[e] + bb[e];
      store4(o + c, y);
    }
  }
}

HB_EXPORT int hb_add_layernorm(void* out, float* residual, const void* a, const float* sa,
                               const void* b, const float* sb, float mult, const float* weight,
                               const float* bias, const int* rows, int n_out, int H, float eps,
                               int act_dt, cudaStream_t stream) {
  if (n_out <= 0) return HB_OK;
  const size_t smem = (size_t)H * sizeof(float);
  if (H <= 0 || smem > 200 * 1024) return HB_BAD_ARGUMENT;
  const bool vec = (H % 4 == 0) && H <= NORM_THREADS * NORM_GROUPS * 4 && ((uintptr_t)out % 16 == 0) &&
                   ((uintptr_t)residual % 16 == 0) && ((uintptr_t)a % 16 == 0) && ((uintptr_t)b % 16 == 0) &&
                   ((uintptr_t)sa % 16 == 0) && ((uintptr_t)sb % 16 == 0) && ((uintptr_t)weight % 16 == 0) &&
                   ((uintptr_t)bias % 16 == 0);
  if (vec) {
    HB_DISPATCH_DTYPE(act_dt, TA,
      hb_launch(add_layernorm_vec_kernel<TA>, dim3(n_out), dim3(NORM_THREADS), 0, stream, (TA*)out, residual,
                (const TA*)a, sa, (const TA*)b, sb, mult, weight, bias, rows, H, eps));
    return hb_check_launch();
  }
  HB_DISPATCH_DTYPE(act_dt, TA,
    if (smem > 40 * 1024)
      cudaFuncSetAttribute(add_layernorm_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    hb_launch(add_layernorm_kernel<TA>, dim3(n_out), dim3(NORM_THREADS), smem, stream, (TA*)out, residual,
              (const TA*)a, sa, (const TA*)b, sb, mult, weight, bias, rows, H, eps));
  return hb_check_launch();
}

// ---------------------------------------------------------------- learned positions
// hidden[t, :] (f32) += table[index[t], :]: a vector per position, added to the embedded token.
template <typename T>
__global__ void add_table_rows_kernel(float* __restrict__ hidden, const T* __restrict__ table,
                                      const int* __restrict__ index, int H, int V) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int id = index[t];
  if (id < 0 || id >= V) id = V - 1;      // positions are bounded on the host
  const T* row = table + (size_t)id * H;
  float* o = hidden + (size_t)t * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) o[i] += to_float(row[i]);
}

HB_EXPORT int hb_add_table_rows(float* hidden, const void* table, const int* index, int T, int H,
                                int V, int table_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  HB_DISPATCH_DTYPE(table_dt, TT,
    hb_launch(add_table_rows_kernel<TT>, dim3(T), dim3(256), 0, stream, hidden, (const TT*)table, index, H, V));
  return hb_check_launch();
}

// ---------------------------------------------------------------- float32 rows into wider act rows
// dst[t, col0 + c] = src[t, c] in the activation dtype (dst has `ld` columns): puts the stream
// beside another tensor as the input of one product.
template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ dst, int ld, int col0, const float* __restrict__ src,
                                 int W, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / W;
    const int c = (int)(idx - t * W);
    dst[t * ld + col0 + c] = from_float<T>(src[idx]);
  }
}

HB_EXPORT int hb_cast_rows(void* dst, int ld, int col0, const float* src, int T, int W, int act_dt,
                           cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (W <= 0 || col0 < 0 || col0 + W > ld) return HB_BAD_ARGUMENT;
  const size_t total = (size_t)T * W;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(cast_rows_kernel<TA>, dim3((unsigned)blocks), dim3(256), 0, stream, (TA*)dst, ld, col0, src, W, total));
  return hb_check_launch();
}

// ---------------------------------------------------------------- q/k norm + cache write
// rows: [T, ld] with q heads (nh * hd), k heads (nkv * hd), v heads (nkv * vd) from column 0.
// One warp per (token, head): a q head becomes q / rms(q) * wq * temp(pos) in place, with
//   temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1)        (every > 0; else 1)
// a k head becomes k / rms(k) * wk at the token's place in its key pages, a v head is copied
// to the value pages.  rms over the head's hd values with eps inside the root; norm weights
// null: no norm.  Pages: [page, kv head, slot, hd] and [page, kv head, slot, vd].  All
// arithmetic float32.  Without `write_cache` k is normed in place and v left alone.
template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_kv_write_kernel(T* __restrict__ rows, int ld, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                        int bt_stride, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens,
                        int nh, int nkv, int hd, int vd, const float* __restrict__ wq,
                        const float* __restrict__ wk, float eps, float coef, int every,
                        int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_token = nh + 2 * nkv;
  const long item = (long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long)n_tokens * per_token) return;
  const int t = (int)(item / per_token), h = (int)(item - (long)t * per_token);
  const int pos = positions[t];
  T* row = rows + (size_t)t * ld;
  size_t page_base = 0;
  int slot = 0;
  if (write_cache && h >= nh) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    slot = pos % page_size;
    page_base = (size_t)page * nkv;
  }
  if (h >= nh + nkv) {                       // a value head
    if (!write_cache) return;
    const int g = h - nh - nkv;
    const T* src = row + (size_t)(nh + nkv) * hd + (size_t)g * vd;
    T* dst = v_pages + ((page_base + g) * page_size + slot) * vd;
    for (int d = lane; d < vd; d += 32) dst[d] = src[d];
    return;
  }
  const bool is_q = h < nh;
  T* x = row + (size_t)h * hd;
  const float* w = is_q ? wq : wk;
  float ss = 0.f;
  for (int d = lane; d < hd; d += 32) { const float v = to_float(x[d]); ss = fmaf(v, v, ss); }
  float f = 1.f;
  if (w) f = rsqrtf(warp_sum(ss) / (float)hd + eps);
  float temp = 1.f;
  if (is_q && every > 0) temp = 1.f + coef * logf((float)((pos + 1) / every) + 1.f);
  T* dst = x;
  if (!is_q && write_cache) dst = k_pages + ((page_base + (h - nh)) * page_size + slot) * hd;
  for (int d = lane; d < hd; d += 32) {
    float v = to_float(x[d]) * f;
    if (w) v *= w[d];
    dst[d] = from_float<T>(v * temp);
  }
}

// The same for bfloat16 rows with 16-byte pieces: a group of hd / 8 lanes (a power of two)
// takes one q or k head, eight values a lane, and sums the squares inside the group; the
// blocks with blockIdx.y == 1 copy the value heads, one 16-byte piece a thread.
template <int GROUP>
__global__ void __launch_bounds__(128)
qk_norm_kv_write_vec_kernel(__nv_bfloat16* __restrict__ rows, int ld, const int* __restrict__ positions,
                            const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                            int bt_stride, __nv_bfloat16* __restrict__ k_pages,
                            __nv_bfloat16* __restrict__ v_pages, int n_tokens, int nh, int nkv, int vd,
                            const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                            float coef, int every, int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int HD = GROUP * 8;
  const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (blockIdx.y == 1) {                       // value heads: pieces of 8 values
    const int per_token = nkv * (vd >> 3);
    if (!write_cache || tid >= (long)n_tokens * per_token) return;
    const int t = (int)(tid / per_token), piece = (int)(tid - (long)t * per_token);
    const int g = piece / (vd >> 3), j = (piece - g * (vd >> 3)) * 8;
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    const __nv_bfloat16* src = rows + (size_t)t * ld + (size_t)(nh + nkv) * HD + (size_t)g * vd + j;
    __nv_bfloat16* dst = v_pages + (((size_t)page * nkv + g) * page_size + pos % page_size) * vd + j;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    return;
  }
  const int per_token = nh + nkv;
  const long item = tid / GROUP;
  const int part = (int)(tid % GROUP);
  const bool live = item < (long)n_tokens * per_token;
  const int t = live ? (int)(item / per_token) : 0, h = live ? (int)(item - (long)t * per_token) : 0;
  const int pos = positions[t];
  const bool is_q = h < nh;
  __nv_bfloat16* x = rows + (size_t)t * ld + (size_t)h * HD + part * 8;
  float v[8];
  {
    float lo[4], hi[4];
    load4(x, lo);
    load4(x + 4, hi);
#pragma unroll
    for (int e = 0; e < 4; ++e) { v[e] = lo[e]; v[4 + e] = hi[e]; }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss = fmaf(v[e], v[e], ss);
#pragma unroll
  for (int o = GROUP / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (!live) return;
  const float* w = is_q ? wq : wk;
  float f = 1.f;
  if (w) f = rsqrtf(ss / (float)HD + eps);
  if (is_q && every > 0) {
    const float temp = 1.f + coef * logf((float)((pos + 1) / every) + 1.f);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float y = v[e] * f;
      if (w) y *= w[part * 8 + e];
      v[e] = y * temp;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float y = v[e] * f;
      if (w) y *= w[part * 8 + e];
      v[e] = y;
    }
  }
  __nv_bfloat16* dst = x;
  if (!is_q && write_cache) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    dst = k_pages + (((size_t)page * nkv + (h - nh)) * page_size + pos % page_size) * HD + part * 8;
  }
  float lo[4] = {v[0], v[1], v[2], v[3]}, hi[4] = {v[4], v[5], v[6], v[7]};
  store4(dst, lo);
  store4(dst + 4, hi);
}

HB_EXPORT int hb_qk_norm_kv_write(void* rows, int ld, const int* positions, const int* seq_of_token,
                                  const int* block_table, int bt_stride, void* k_pages, void* v_pages,
                                  int T, int nh, int nkv, int hd, int vd, const float* wq,
                                  const float* wk, float eps, float coef, int every, int page_size,
                                  int write_cache, int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (nh <= 0 || nkv <= 0 || hd <= 0 || vd <= 0 || page_size <= 0 || every < 0 ||
      (long)nh * hd + (long)nkv * (hd + vd) > ld)
    return HB_BAD_ARGUMENT;
  const int group = hd / 8;
  const bool vec = act_dt == HB_BF16 && hd % 8 == 0 && vd % 8 == 0 && ld % 8 == 0 &&
                   (group == 4 || group == 8 || group == 16 || group == 32) &&
                   (uintptr_t)rows % 16 == 0 && (uintptr_t)k_pages % 16 == 0 && (uintptr_t)v_pages % 16 == 0;
  if (vec) {
    const long norm_threads = (long)T * (nh + nkv) * group;
    const long copy_threads = write_cache ? (long)T * nkv * (vd / 8) : 0;
    const long most = norm_threads > copy_threads ? norm_threads : copy_threads;
    dim3 grid((unsigned)((most + 127) / 128), write_cache ? 2 : 1);
#define HB_QK_VEC(G)                                                                               \
    hb_launch(qk_norm_kv_write_vec_kernel<G>, grid, dim3(128), 0, stream, (__nv_bfloat16*)rows, ld,   \
              positions, seq_of_token, block_table, bt_stride, (__nv_bfloat16*)k_pages,               \
              (__nv_bfloat16*)v_pages, T, nh, nkv, vd, wq, wk, eps, coef, every, page_size, write_cache)
    if (group == 4) HB_QK_VEC(4);
    else if (group == 8) HB_QK_VEC(8);
    else if (group == 16) HB_QK_VEC(16);
    else HB_QK_VEC(32);
#undef HB_QK_VEC
    return hb_check_launch();
  }
  const long items = (long)T * (nh + 2 * nkv);
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(qk_norm_kv_write_kernel<TA>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, stream, (TA*)rows, ld,
              positions, seq_of_token, block_table, bt_stride, (TA*)k_pages, (TA*)v_pages, T, nh, nkv,
              hd, vd, wq, wk, eps, coef, every, page_size, write_cache));
  return hb_check_launch();
}

// ---------------------------------------------------------------- rotation, q/k norm, cache write
// rows: [T, ld] with q heads (nh * hd) from column 0, then k heads (nkv * hd); value heads
// (nkv * vd) at column v_col, or, with v_col < 0, the values ARE the keys as projected (before
// rotation and norm; vd = hd).  One warp per (token, head):
//   a q or k head is rotated on its first `rot` values ((u, v) -> (u cos - v sin, v cos + u sin),
//   cos/sin [T, rot/2] float32; rot 0: none; `pairing` QKR_HALVES: value i paired with value
//   i + rot/2, QKR_NEIGHBOURS: value 2i with value 2i + 1), then, with `norm` QKR_NORM_HEAD,
//   divided by its root mean square over hd (eps inside the root) and multiplied by a weight per
//   channel (wq / wk [hd], null: none);
//   with `norm` QKR_NORM_ROW the norm comes BEFORE the rotation and runs over the whole q row
//   (nh * hd values) and the whole k row (nkv * hd) at once, with weights wq [nh * hd] and
//   wk [nkv * hd]: one block a token takes the two sums first and then walks the heads;
//   q is written back in place; k goes to the token's place in the key pages, the values to
//   the value pages (pages: [page, kv head, slot, hd] and [.., vd]).
// All arithmetic float32.  Without `write_cache` k is written back in place and no value moves.
constexpr int QKR_WARPS = 4;
constexpr int QKR_ROW_WARPS = 8;
constexpr int QKR_MAX_HD = 256;
enum { QKR_HALVES = 0, QKR_NEIGHBOURS = 1 };
enum { QKR_NORM_NONE = 0, QKR_NORM_HEAD = 1, QKR_NORM_ROW = 2 };

// head h of token t by one warp; `xs`: hd floats of shared memory of the warp's own.
// row_f: QKR_NORM_ROW: 1 / rms of the head's whole row (q or k); else unused.
template <typename T>
__device__ __forceinline__ void
qkr_head(T* __restrict__ rows, int ld, int v_col, const float* __restrict__ cos_tab,
         const float* __restrict__ sin_tab, int rot, int pairing, const int* __restrict__ positions,
         const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int bt_stride,
         T* __restrict__ k_pages, T* __restrict__ v_pages, int nh, int nkv, int hd, int vd, int norm,
         const float* __restrict__ wq, const float* __restrict__ wk, float eps, int page_size,
         int write_cache, int t, int h, float* xs, int lane, float row_f) {
  const int pos = positions[t];
  T* row = rows + (size_t)t * ld;
  size_t page_base = 0;
  int slot = 0;
  if (write_cache && h >= nh) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    slot = pos % page_size;
    page_base = (size_t)page * nkv;
  }
  if (h >= nh + nkv) {                       // a value head with columns of its own
    if (!write_cache) return;
    const int g = h - nh - nkv;
    const T* src = row + v_col + (size_t)g * vd;
    T* dst = v_pages + ((page_base + g) * page_size + slot) * vd;
    for (int d = lane; d < vd; d += 32) dst[d] = src[d];
    return;
  }
  const bool is_q = h < nh;
  T* x = row + (size_t)h * hd;
  const float* w = is_q ? wq : wk;
  // the norm over the whole row: its factor and the channel's weight go on before the rotation
  const float* w_pre = (norm == QKR_NORM_ROW && w) ? w + (size_t)(is_q ? h : h - nh) * hd : nullptr;
  const float f_pre = norm == QKR_NORM_ROW ? row_f : 1.f;
  if (!is_q && write_cache && v_col < 0) {   // the values are the keys as projected
    T* dst = v_pages + ((page_base + (h - nh)) * page_size + slot) * vd;
    for (int d = lane; d < hd; d += 32) { const T v = x[d]; dst[d] = v; xs[d] = to_float(v); }
  } else {
    for (int d = lane; d < hd; d += 32) xs[d] = to_float(x[d]);
  }
  if (norm == QKR_NORM_ROW)
    for (int d = lane; d < hd; d += 32) xs[d] = xs[d] * f_pre * (w_pre ? w_pre[d] : 1.f);
  __syncwarp();
  const int half = rot >> 1;
  const float* cr = cos_tab ? cos_tab + (size_t)t * half : nullptr;
  const float* sr = sin_tab ? sin_tab + (size_t)t * half : nullptr;
  constexpr int PER = QKR_MAX_HD / 32;
  float y[PER];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = lane + 32 * i;
    float v = 0.f;
    if (d < hd) {
      v = xs[d];
      if (d < rot) {
        if (pairing == QKR_NEIGHBOURS) {
          const float c = cr[d >> 1], s = sr[d >> 1];
          v = (d & 1) ? v * c + xs[d - 1] * s : v * c - xs[d + 1] * s;
        } else {
          const int j = d < half ? d : d - half;
          const float c = cr[j], s = sr[j];
          v = d < half ? v * c - xs[d + half] * s : v * c + xs[d - half] * s;
        }
      }
    }
    y[i] = v;
    ss = fmaf(v, v, ss);
  }
  float f = 1.f;
  if (norm == QKR_NORM_HEAD) f = rsqrtf(warp_sum(ss) / (float)hd + eps);
  T* dst = x;
  if (!is_q && write_cache) dst = k_pages + ((page_base + (h - nh)) * page_size + slot) * hd;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) {
      float v = y[i] * f;
      if (norm == QKR_NORM_HEAD && w) v *= w[d];
      dst[d] = from_float<T>(v);
    }
  }
  __syncwarp();                               // xs may serve the warp's next head
}

template <typename T>
__global__ void __launch_bounds__(QKR_WARPS * 32)
qk_rotate_norm_write_kernel(T* __restrict__ rows, int ld, int v_col, const float* __restrict__ cos_tab,
                            const float* __restrict__ sin_tab, int rot, int pairing,
                            const int* __restrict__ positions,
                            const int* __restrict__ seq_of_token, const int* __restrict__ block_table,
                            int bt_stride, T* __restrict__ k_pages, T* __restrict__ v_pages, int n_tokens,
                            int nh, int nkv, int hd, int vd, int norm, const float* __restrict__ wq,
                            const float* __restrict__ wk, float eps, int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float head_sm[QKR_WARPS][QKR_MAX_HD];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int per_token = nh + nkv + (v_col >= 0 ? nkv : 0);
  const long item = (long)blockIdx.x * QKR_WARPS + warp;
  if (item >= (long)n_tokens * per_token) return;
  const int t = (int)(item / per_token), h = (int)(item - (long)t * per_token);
  qkr_head<T>(rows, ld, v_col, cos_tab, sin_tab, rot, pairing, positions, seq_of_token, block_table, bt_stride,
              k_pages, v_pages, nh, nkv, hd, vd, norm, wq, wk, eps, page_size, write_cache, t, h,
              head_sm[warp], lane, 1.f);
}

// The norm over whole rows: one block a token.  The sums of squares of the q row and of the
// k row are taken by all threads in an order that depends on the row alone; then every warp
// walks heads warp, warp + QKR_ROW_WARPS, ...
template <typename T>
__global__ void __launch_bounds__(QKR_ROW_WARPS * 32)
qk_rownorm_rotate_write_kernel(T* __restrict__ rows, int ld, int v_col, const float* __restrict__ cos_tab,
                               const float* __restrict__ sin_tab, int rot, int pairing,
                               const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                               const int* __restrict__ block_table, int bt_stride, T* __restrict__ k_pages,
                               T* __restrict__ v_pages, int nh, int nkv, int hd, int vd,
                               const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                               int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float head_sm[QKR_ROW_WARPS][QKR_MAX_HD];
  __shared__ float scratch[33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* row = rows + (size_t)t * ld;
  const int nq = nh * hd, nk = nkv * hd;
  float sq = 0.f, sk = 0.f;
  for (int c = threadIdx.x; c < nq; c += blockDim.x) { const float v = to_float(row[c]); sq = fmaf(v, v, sq); }
  for (int c = threadIdx.x; c < nk; c += blockDim.x) { const float v = to_float(row[nq + c]); sk = fmaf(v, v, sk); }
  const float fq = rsqrtf(block_sum(sq, scratch) / (float)nq + eps);
  const float fk = rsqrtf(block_sum(sk, scratch) / (float)nk + eps);
  const int per_token = nh + nkv + (v_col >= 0 ? nkv : 0);
  for (int h = warp; h < per_token; h += QKR_ROW_WARPS)
    qkr_head<T>(const_cast<T*>(rows), ld, v_col, cos_tab, sin_tab, rot, pairing, positions, seq_of_token,
                block_table, bt_stride, k_pages, v_pages, nh, nkv, hd, vd, QKR_NORM_ROW, wq, wk, eps,
                page_size, write_cache, t, h, head_sm[warp], lane, h < nh ? fq : fk);
}

// The same with 16-byte pieces, for rows whose heads, strides and offsets are whole pieces (8
// bfloat16 or 4 float32 values): the q and k rows pass through shared memory as floats once;
// the sums of squares are taken while they are loaded (a thread's pieces in their order, then
// the block's fixed tree); after ONE barrier every thread norms, weights and rotates pieces
// (a neighbour pair lies inside a piece; the partner of a halves pair is read from shared
// memory with its own weight) and stores them whole; value heads are copied piece by piece.
constexpr int QKR_FAST_THREADS = 128;

template <typename T>
__global__ void __launch_bounds__(QKR_FAST_THREADS)
qk_rownorm_rotate_write_vec_kernel(T* __restrict__ rows, int ld, int v_col, const float* __restrict__ cos_tab,
                                   const float* __restrict__ sin_tab, int rot, int pairing,
                                   const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                   const int* __restrict__ block_table, int bt_stride, T* __restrict__ k_pages,
                                   T* __restrict__ v_pages, int nh, int nkv, int hd, int vd,
                                   const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                   int page_size, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int V = 16 / sizeof(T);
  extern __shared__ float qkr_sm[];            // [nq + nk] the rows as floats, then 66 floats of scratch
  const int t = blockIdx.x, tid = threadIdx.x;
  const int nq = nh * hd, nk = nkv * hd, n = nq + nk;
  float* scratch = qkr_sm + n;
  T* row = rows + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int c = tid * V; c < n; c += QKR_FAST_THREADS * V) {
    const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
    const T* e = reinterpret_cast<const T*>(&raw);
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < V; ++i) { const float v = to_float(e[i]); qkr_sm[c + i] = v; part = fmaf(v, v, part); }
    if (c < nq) sq += part; else sk += part;
  }
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if ((tid & 31) == 0) { scratch[tid >> 5] = sq; scratch[32 + (tid >> 5)] = sk; }
  __syncthreads();
  float tq = 0.f, tk = 0.f;
#pragma unroll
  for (int w = 0; w < QKR_FAST_THREADS / 32; ++w) { tq += scratch[w]; tk += scratch[32 + w]; }
  const float fq = rsqrtf(tq / (float)nq + eps), fk = rsqrtf(tk / (float)nk + eps);
  const int pos = positions[t];
  size_t page_base = 0;
  int slot = 0;
  if (write_cache) {
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    slot = pos % page_size;
    page_base = (size_t)page * nkv;
  }
  const int half = rot >> 1;
  const float* cr = cos_tab ? cos_tab + (size_t)t * half : nullptr;
  const float* sr = sin_tab ? sin_tab + (size_t)t * half : nullptr;
  for (int c = tid * V; c < n; c += QKR_FAST_THREADS * V) {
    const bool is_q = c < nq;
    const int cc = is_q ? c : c - nq;                 // column inside the q or the k row
    const int h = cc / hd, d0 = cc - h * hd;
    const float f = is_q ? fq : fk;
    const float* w = is_q ? wq : wk;
    const float* x = qkr_sm + c;
    float y[V];
#pragma unroll
    for (int i = 0; i < V; ++i) y[i] = x[i] * f * (w ? w[cc + i] : 1.f);
    if (!is_q && write_cache && v_col < 0) {          // the values are the keys as projected
      uint4 out;
      T* o = reinterpret_cast<T*>(&out);
#pragma unroll
      for (int i = 0; i < V; ++i) o[i] = from_float<T>(x[i]);
      *reinterpret_cast<uint4*>(v_pages + ((page_base + h) * page_size + slot) * vd + d0) = out;
    }
    if (d0 < rot) {
      if (pairing == QKR_NEIGHBOURS) {
#pragma unroll
        for (int i = 0; i < V; i += 2) {
          if (d0 + i < rot) {
            const float co = cr[(d0 + i) >> 1], si = sr[(d0 + i) >> 1];
            const float u = y[i], v = y[i + 1];
            y[i] = u * co - v * si;
            y[i + 1] = v * co + u * si;
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          const int d = d0 + i;
          if (d < rot) {
            const bool low = d < half;
            const int j = low ? d : d - half, pd = low ? d + half : d - half;
            const float partner = qkr_sm[c - d0 + pd] * f * (w ? w[cc - d0 + pd] : 1.f);
            y[i] = low ? y[i] * cr[j] - partner * sr[j] : y[i] * cr[j] + partner * sr[j];
          }
        }
      }
    }
    uint4 out;
    T* o = reinterpret_cast<T*>(&out);
#pragma unroll
    for (int i = 0; i < V; ++i) o[i] = from_float<T>(y[i]);
    T* dst = (!is_q && write_cache) ? k_pages + ((page_base + h) * page_size + slot) * hd + d0 : row + c;
    *reinterpret_cast<uint4*>(dst) = out;
  }
  if (write_cache && v_col >= 0) {
    const int nv = nkv * vd;
    for (int c = tid * V; c < nv; c += QKR_FAST_THREADS * V) {
      const int g = c / vd, d0 = c - g * vd;
      *reinterpret_cast<uint4*>(v_pages + ((page_base + g) * page_size + slot) * vd + d0) =
          *reinterpret_cast<const uint4*>(row + v_col + c);
    }
  }
}

HB_EXPORT int hb_qk_rotate_norm_write(void* rows, int ld, int v_col, const float* cos_tab,
                                      const float* sin_tab, int rot, int pairing, const int* positions,
                                      const int* seq_of_token, const int* block_table, int bt_stride,
                                      void* k_pages, void* v_pages, int T, int nh, int nkv, int hd, int vd,
                                      int norm, const float* wq, const float* wk, float eps, int page_size,
                                      int write_cache, int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (nh <= 0 || nkv <= 0 || hd <= 0 || hd > QKR_MAX_HD || vd <= 0 || page_size <= 0 || rot < 0 ||
      rot > hd || rot % 2 || (rot > 0 && (cos_tab == nullptr || sin_tab == nullptr)) ||
      (pairing != QKR_HALVES && pairing != QKR_NEIGHBOURS) || norm < QKR_NORM_NONE || norm > QKR_NORM_ROW ||
      (v_col < 0 && vd != hd) || (long)(nh + nkv) * hd > ld || (v_col >= 0 && (long)v_col + (long)nkv * vd > ld))
    return HB_BAD_ARGUMENT;
  if (norm == QKR_NORM_ROW) {
    // 16-byte pieces where every head, stride and offset is a whole number of them
    const int V = act_dt == HB_BF16 ? 8 : 4;
    const size_t smem = ((size_t)(nh + nkv) * hd + 66) * sizeof(float);
    const uintptr_t bits = reinterpret_cast<uintptr_t>(rows) | reinterpret_cast<uintptr_t>(k_pages) |
                           reinterpret_cast<uintptr_t>(v_pages);
    if (hd % V == 0 && vd % V == 0 && ld % V == 0 && (v_col < 0 || v_col % V == 0) && (bits & 15) == 0 &&
        smem <= 200 * 1024) {
      HB_DISPATCH_DTYPE(act_dt, TA, {
        if (smem > 48 * 1024)
          cudaFuncSetAttribute(qk_rownorm_rotate_write_vec_kernel<TA>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               (int)smem);
        hb_launch(qk_rownorm_rotate_write_vec_kernel<TA>, dim3((unsigned)T), dim3(QKR_FAST_THREADS), smem, stream,
                  (TA*)rows, ld, v_col, cos_tab, sin_tab, rot, pairing, positions, seq_of_token, block_table,
                  bt_stride, (TA*)k_pages, (TA*)v_pages, nh, nkv, hd, vd, wq, wk, eps, page_size, write_cache);
      });
      return hb_check_launch();
    }
    HB_DISPATCH_DTYPE(act_dt, TA,
      hb_launch(qk_rownorm_rotate_write_kernel<TA>, dim3((unsigned)T), dim3(QKR_ROW_WARPS * 32), 0, stream,
                (TA*)rows, ld, v_col, cos_tab, sin_tab, rot, pairing, positions, seq_of_token, block_table,
                bt_stride, (TA*)k_pages, (TA*)v_pages, nh, nkv, hd, vd, wq, wk, eps, page_size, write_cache));
    return hb_check_launch();
  }
  const long items = (long)T * (nh + nkv + (v_col >= 0 ? nkv : 0));
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(qk_rotate_norm_write_kernel<TA>, dim3((unsigned)((items + QKR_WARPS - 1) / QKR_WARPS)),
              dim3(QKR_WARPS * 32), 0, stream, (TA*)rows, ld, v_col, cos_tab, sin_tab, rot, pairing, positions,
              seq_of_token, block_table, bt_stride, (TA*)k_pages, (TA*)v_pages, T, nh, nkv, hd, vd, norm,
              wq, wk, eps, page_size, write_cache));
  return hb_check_launch();
}

// ---------------------------------------------------------------- activations of one argument
// out = act(x), element by element, float32 arithmetic: 0 the square of relu, 1 silu,
// 2 gelu (tanh form), 3 x * sigmoid(gate) with `gate` [T, >= W] rows gate_ld apart.
enum { ACT_RELU2 = 0, ACT_SILU = 1, ACT_GELU_TANH = 2, ACT_SIGMOID_GATE = 3 };

template <typename T>
__global__ void unary_act_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ gate,
                                 int gate_ld, size_t total, int W, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const float v = to_float(x[idx]);
    float y;
    if (kind == ACT_RELU2) { const float r = fmaxf(v, 0.f); y = r * r; }
    else if (kind == ACT_SILU) y = v / (1.f + expf(-v));
    else if (kind == ACT_GELU_TANH) y = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
    else {
      const size_t t = idx / W;
      const float g = to_float(gate[t * (size_t)gate_ld + (idx - t * W)]);
      y = v / (1.f + expf(-g));
    }
    out[idx] = from_float<T>(y);
  }
}

// bfloat16 rows whose values come in 16-byte pieces: eight values a thread and step.
__global__ void unary_act_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                                        size_t pieces, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < pieces;
       idx += (size_t)gridDim.x * blockDim.x) {
    const uint4 raw = reinterpret_cast<const uint4*>(x)[idx];
    const uint32_t in[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t res[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&in[e]));
      float y[2];
#pragma unroll
      for (int k = 0; k < 2; ++k) {
        const float u = k ? v.y : v.x;
        if (kind == ACT_RELU2) { const float r = fmaxf(u, 0.f); y[k] = r * r; }
        else if (kind == ACT_SILU) y[k] = u / (1.f + expf(-u));
        else y[k] = 0.5f * u * (1.f + tanhf(0.7978845608028654f * (u + 0.044715f * u * u * u)));
      }
      const __nv_bfloat162 o = __floats2bfloat162_rn(y[0], y[1]);
      res[e] = *reinterpret_cast<const uint32_t*>(&o);
    }
    reinterpret_cast<uint4*>(out)[idx] = make_uint4(res[0], res[1], res[2], res[3]);
  }
}

HB_EXPORT int hb_unary_act(void* out, const void* x, const void* gate, int gate_ld, int T, int W, int kind,
                           int act_dt, cudaStream_t stream) {
  if (T <= 0 || W <= 0) return HB_OK;
  if (kind < 0 || kind > 3 || (kind == ACT_SIGMOID_GATE && gate == nullptr)) return HB_BAD_ARGUMENT;
  const size_t total = (size_t)T * W;
  if (act_dt == HB_BF16 && kind != ACT_SIGMOID_GATE && total % 8 == 0 &&
      ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x)) & 15) == 0) {
    const size_t pieces = total / 8;
    size_t vblocks = (pieces + 255) / 256;
    if (vblocks > 148 * 16) vblocks = 148 * 16;
    hb_launch(unary_act_bf16x8_kernel, dim3((unsigned)vblocks), dim3(256), 0, stream, (__nv_bfloat16*)out,
              (const __nv_bfloat16*)x, pieces, kind);
    return hb_check_launch();
  }
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(unary_act_kernel<TA>, dim3((unsigned)blocks), dim3(256), 0, stream, (TA*)out, (const TA*)x,
              (const TA*)gate, gate_ld, total, W, kind));
  return hb_check_launch();
}

// ---------------------------------------------------------------- a gate on every value of every head
// out[t, h * N + n] = x[t, h, n] * sigmoid(gate[t, h * N + n]): x is a view [T, H, N] with a
// token stride and a head stride (what a batched product of one matrix a head leaves), gate rows
// are gate_ld apart, out is contiguous.  float32 arithmetic.
template <typename T>
__global__ void gate_heads_kernel(T* __restrict__ out, const T* __restrict__ x, long x_token, long x_head,
                                  const T* __restrict__ gate, int gate_ld, size_t total, int H, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int W = H * N;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / W;
    const int c = (int)(idx - t * W), h = c / N, n = c - h * N;
    const float v = to_float(x[t * x_token + (size_t)h * x_head + n]);
    const float g = to_float(gate[t * (size_t)gate_ld + c]);
    out[idx] = from_float<T>(v / (1.f + expf(-g)));
  }
}

// bfloat16, N a multiple of 8 and every row 16-byte aligned: eight values a thread and step
__global__ void gate_heads_bf16x8_kernel(__nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ x,
                                         long x_token, long x_head, const __nv_bfloat16* __restrict__ gate,
                                         int gate_ld, size_t pieces, int H, int N) {
  pdl_launch_dependents();
  pdl_wait();
  const int W8 = H * N / 8, N8 = N / 8;
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < pieces;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / W8;
    const int c = (int)(idx - t * W8), h = c / N8, n = (c - h * N8) * 8;
    const uint4 xv = *reinterpret_cast<const uint4*>(x + t * x_token + (size_t)h * x_head + n);
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + t * (size_t)gate_ld + (size_t)c * 8);
    const __nv_bfloat162* xp = reinterpret_cast<const __nv_bfloat162*>(&xv);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gv);
    uint4 ov;
    __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 a = __bfloat1622float2(xp[i]), g = __bfloat1622float2(gp[i]);
      op[i] = __floats2bfloat162_rn(a.x / (1.f + expf(-g.x)), a.y / (1.f + expf(-g.y)));
    }
    *reinterpret_cast<uint4*>(out + idx * 8) = ov;
  }
}

HB_EXPORT int hb_gate_heads(void* out, const void* x, long x_token, long x_head, const void* gate, int gate_ld,
                            int T, int H, int N, int act_dt, cudaStream_t stream) {
  if (T <= 0 || H <= 0 || N <= 0) return HB_OK;
  if (gate == nullptr || gate_ld < H * N) return HB_BAD_ARGUMENT;
  const size_t total = (size_t)T * H * N;
  const bool aligned = ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(x) |
                         reinterpret_cast<uintptr_t>(gate)) & 15) == 0;
  if (act_dt == HB_BF16 && N % 8 == 0 && x_token % 8 == 0 && x_head % 8 == 0 && gate_ld % 8 == 0 && aligned) {
    const size_t pieces = total / 8;
    size_t blocks = (pieces + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    hb_launch(gate_heads_bf16x8_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, (__nv_bfloat16*)out,
              (const __nv_bfloat16*)x, x_token, x_head, (const __nv_bfloat16*)gate, gate_ld, pieces, H, N);
    return hb_check_launch();
  }
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(gate_heads_kernel<TA>, dim3((unsigned)blocks), dim3(256), 0, stream, (TA*)out, (const TA*)x,
              x_token, x_head, (const TA*)gate, gate_ld, total, H, N));
  return hb_check_launch();
}

