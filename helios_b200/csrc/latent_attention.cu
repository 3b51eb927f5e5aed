// Attention over a cache of latents: every token stores ONE row [c | r] (c: `rank` values,
// the normed low-rank latent; r: `rot` values, a rotated key part shared by all heads)
// instead of keys and values per head.  With the per-head up-projections folded into
// the query and the output (q_lat[h] = W_uk[h]^T q[h], o[h] = W_uv[h] o_lat[h]) every
// head attends the same rows:
//
//   score(t, h, j) = (q_lat[t, h] . c_j + q_rot[t, h] . r_j) * scale
//   o_lat[t, h]    = sum_j softmax_j(score) c_j
//
// Three kernels: `latent_prepare` (RMS norm of the latent, rotary on the shared key part
// and on the queries' rotated parts, cache write), `head_gemm` (the folded products, one
// small matrix per head) and `latent_attention` (one warp per (token, head), float32
// scores, softmax and sums, keys walked in runs of 32 from position 0 so that the order
// of every sum depends on the token's position alone).
#include "common.cuh"

// ---------------------------------------------------------------- prepare
// What the rows of the projections want before attention; every piece is optional (a null
// pointer leaves it out), one block a token:
//   cq  [T, cq_ld]: a query latent of `q_rank` values, RMS-normed (weight cq_w) into cq_out
//       [T, cq_out_ld] (which may be cq itself: in place);
//   lat [T, lat_ld] = [latent (rank) | shared key part (rot)]: the latent RMS-normed (weight
//       norm_w), the shared key part rotated, both stored as the token's row of `pages`
//       (with `write_cache`; without it nothing of `lat` is used: another layer's rows serve);
//   q   [T, q_ld] = heads x [nope | rot]: every head's rotated part rotated in place.
// The rotation runs over the first `nrot` of the `rot` values; `pairing` 0: value i with value
// i + nrot / 2 (halves), 1: value 2i with value 2i + 1 (neighbours); cos/sin tables are
// [T, nrot / 2] (any factor already in them).  float32 arithmetic, eps inside the roots.
enum { LAT_HALVES = 0, LAT_NEIGHBOURS = 1 };

template <typename T>
__device__ __forceinline__ void latent_rotate(T* __restrict__ dst, const T* __restrict__ src, int i, int half,
                                              int pairing, const float* __restrict__ ct,
                                              const float* __restrict__ st) {
  const int a = pairing == LAT_NEIGHBOURS ? 2 * i : i;
  const int b = pairing == LAT_NEIGHBOURS ? 2 * i + 1 : i + half;
  const float u = to_float(src[a]), v = to_float(src[b]);
  dst[a] = from_float<T>(u * ct[i] - v * st[i]);
  dst[b] = from_float<T>(v * ct[i] + u * st[i]);
}

template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(T* __restrict__ q, int q_ld, const T* __restrict__ lat_rows, int lat_ld,
                      const T* cq, int cq_ld, T* cq_out, int cq_out_ld, int q_rank,
                      const float* __restrict__ cq_w,
                      T* __restrict__ pages, const float* __restrict__ norm_w,
                      const float* __restrict__ cos_tab, const float* __restrict__ sin_tab,
                      const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                      const int* __restrict__ block_table, int bt_stride, int heads, int nope, int rot,
                      int rank, int nrot, int pairing, int page_size, float eps, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const int half = nrot / 2;
  const float* ct = cos_tab + (size_t)t * half;
  const float* st = sin_tab + (size_t)t * half;
  if (cq) {                                  // the query latent, normed in float32
    const T* row = cq + (size_t)t * cq_ld;
    T* out = cq_out + (size_t)t * cq_out_ld;
    float ss = 0.f;
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x) { const float v = to_float(row[c]); ss += v * v; }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)q_rank + eps);
    for (int c = threadIdx.x; c < q_rank; c += blockDim.x)
      out[c] = from_float<T>(to_float(row[c]) * rstd * cq_w[c]);
  }
  if (lat_rows && write_cache) {
    const T* lat = lat_rows + (size_t)t * lat_ld;
    const int pos = positions[t];
    const int page = block_table[(size_t)seq_of_token[t] * bt_stride + pos / page_size];
    T* dst = pages + ((size_t)page * page_size + pos % page_size) * (rank + rot);
    // the latent, normed in float32
    float ss = 0.f;
    for (int c = threadIdx.x; c < rank; c += blockDim.x) { const float v = to_float(lat[c]); ss += v * v; }
    const float rstd = rsqrtf(block_sum(ss, scratch) / (float)rank + eps);
    for (int c = threadIdx.x; c < rank; c += blockDim.x)
      dst[c] = from_float<T>(to_float(lat[c]) * rstd * norm_w[c]);
    // the shared key part: rotated pairs, the rest as it is
    const T* kr = lat + rank;
    for (int i = threadIdx.x; i < half; i += blockDim.x) latent_rotate(dst + rank, kr, i, half, pairing, ct, st);
    for (int c = nrot + threadIdx.x; c < rot; c += blockDim.x) dst[rank + c] = kr[c];
  }
  if (q) {                                   // the queries' rotated parts, in place
    T* row = q + (size_t)t * q_ld;
    for (int idx = threadIdx.x; idx < heads * half; idx += blockDim.x) {
      const int h = idx / half, i = idx - h * half;
      T* qr = row + (size_t)h * (nope + rot) + nope;
      latent_rotate(qr, qr, i, half, pairing, ct, st);
    }
  }
}

HB_EXPORT int hb_latent_prepare(void* q, int q_ld, const void* lat, int lat_ld, const void* cq, int cq_ld,
                                void* cq_out, int cq_out_ld, int q_rank, const float* cq_w, void* pages,
                                const float* norm_w,
                                const float* cos_tab, const float* sin_tab, const int* positions,
                                const int* seq_of_token, const int* block_table, int bt_stride,
                                int T, int heads, int nope, int rot, int rank, int nrot, int pairing,
                                int page_size, float eps, int write_cache, int act_dt,
                                cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (heads <= 0 || nope < 0 || rot < 0 || rank <= 0 || nrot < 0 || nrot > rot || nrot % 2 ||
      page_size <= 0 || (pairing != LAT_HALVES && pairing != LAT_NEIGHBOURS) ||
      (q && q_ld < heads * (nope + rot)) || (lat && lat_ld < rank + rot) ||
      (cq && (q_rank <= 0 || cq_ld < q_rank || cq_w == nullptr || cq_out == nullptr || cq_out_ld < q_rank)) ||
      (lat && write_cache && (pages == nullptr || norm_w == nullptr)) ||
      (nrot > 0 && (cos_tab == nullptr || sin_tab == nullptr)))
    return HB_BAD_ARGUMENT;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(latent_prepare_kernel<TA>, dim3(T), dim3(128), 0, stream, (TA*)q, q_ld, (const TA*)lat, lat_ld,
              (const TA*)cq, cq_ld, (TA*)cq_out, cq_out_ld, q_rank, cq_w, (TA*)pages, norm_w, cos_tab, sin_tab, positions, seq_of_token,
              block_table, bt_stride, heads, nope, rot, rank, nrot, pairing, page_size, eps, write_cache));
  return hb_check_launch();
}

// ---------------------------------------------------------------- one small matrix per head
// C[m, b, n] = sum_k A[m, b, k] * W[b, n, k] for b < batch: rows of A, W and C have strides,
// and so have the batches.  float32 sums, every element summed over k = 0..K-1 in that
// order in one thread, so a row's result does not depend on the other rows.
constexpr int HG_BM = 64, HG_BN = 64, HG_BK = 16;

template <typename T>
__global__ void __launch_bounds__(256)
head_gemm_kernel(T* __restrict__ C, const T* __restrict__ A, const T* __restrict__ W, int M, int N,
                 int K, long lda, long ldw, long ldc, long a_batch, long w_batch, long c_batch) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float As[HG_BK][HG_BM + 4];
  __shared__ float Ws[HG_BK][HG_BN + 4];
  A += (size_t)blockIdx.z * a_batch;
  W += (size_t)blockIdx.z * w_batch;
  C += (size_t)blockIdx.z * c_batch;
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * HG_BM, n0 = blockIdx.x * HG_BN;
  const int tx = tid & 15, ty = tid >> 4;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  for (int k0 = 0; k0 < K; k0 += HG_BK) {
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int k = k0 + lk + e;
      const int am = m0 + lrow, wn = n0 + lrow;
      As[lk + e][lrow] = (am < M && k < K) ? to_float(A[(size_t)am * lda + k]) : 0.f;
      Ws[lk + e][lrow] = (wn < N && k < K) ? to_float(W[(size_t)wn * ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HG_BK; ++k) {
      float a[4], w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) C[(size_t)m * ldc + n] = from_float<T>(acc[i][j]);
    }
  }
}

HB_EXPORT int hb_head_gemm(void* C, const void* A, const void* W, int M, int N, int K, long lda,
                           long ldw, long ldc, int batch, long a_batch, long w_batch, long c_batch,
                           int act_dt, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || batch <= 0) return HB_OK;
  if (K <= 0 || batch > 65535) return HB_BAD_ARGUMENT;
  dim3 grid((N + HG_BN - 1) / HG_BN, (M + HG_BM - 1) / HG_BM, batch);
  if (grid.y > 65535) return HB_BAD_ARGUMENT;
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(head_gemm_kernel<TA>, grid, dim3(256), 0, stream, (TA*)C, (const TA*)A, (const TA*)W,
              M, N, K, lda, ldw, ldc, a_batch, w_batch, c_batch));
  return hb_check_launch();
}

// ---------------------------------------------------------------- attention
constexpr int LA_WARPS = 4;
constexpr int LA_MAX_RANK = 512;     // latent values a lane accumulates: 16 x 32
constexpr int LA_MAX_ROW = 1024;     // rank + rot

// q_lat[t, h] at q_lat + t * ql_t + h * ql_h (rank values); q_rot likewise (rot values).
// out [T, heads, rank], contiguous.
template <typename T>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attention_kernel(T* __restrict__ out, const T* __restrict__ q_lat, long ql_t, long ql_h,
                        const T* __restrict__ q_rot, long qr_t, long qr_h,
                        const T* __restrict__ pages, const int* __restrict__ block_table,
                        int bt_stride, const int* __restrict__ seq_of_token,
                        const int* __restrict__ positions, int n_rows, int heads, int rank, int rot,
                        int page_size, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float q_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * LA_WARPS + warp;
  if (row >= n_rows) return;
  const int t = row / heads, h = row - t * heads;
  const int width = rank + rot;
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * bt_stride;

  float* qs = q_smem + (size_t)warp * width;
  const T* ql = q_lat + (size_t)t * ql_t + (size_t)h * ql_h;
  const T* qr = q_rot + (size_t)t * qr_t + (size_t)h * qr_h;
  for (int d = lane; d < rank; d += 32) qs[d] = to_float(ql[d]);
  for (int d = lane; d < rot; d += 32) qs[rank + d] = to_float(qr[d]);
  __syncwarp();

  constexpr int ND = LA_MAX_RANK / 32;
  float acc[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = 0; base <= pos; base += 32) {
    const int key = base + lane;
    const bool valid = key <= pos;
    int page = 0;
    float score = -INFINITY;
    if (valid) {
      page = table[key / page_size];
      const T* kr = pages + ((size_t)page * page_size + key % page_size) * width;
      float dot = 0.f;
      for (int d = 0; d < width; ++d) dot = fmaf(qs[d], to_float(kr[d]), dot);
      score = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(score));
    const float p = valid ? expf(score - m_new) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : expf(m - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= corr;
    const int n_valid = min(32, pos - base + 1);
    for (int j = 0; j < n_valid; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const int pagej = __shfl_sync(0xffffffffu, page, j);
      const T* vr = pages + ((size_t)pagej * page_size + (base + j) % page_size) * width;
#pragma unroll
      for (int i = 0; i < ND; ++i) {
        const int d = lane + 32 * i;
        if (d < rank) acc[i] = fmaf(pj, to_float(vr[d]), acc[i]);
      }
    }
  }
  const float inv = 1.f / l;
  T* orow = out + ((size_t)t * heads + h) * rank;
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
    if (d < rank) orow[d] = from_float<T>(acc[i] * inv);
  }
}

HB_EXPORT int hb_latent_attention(void* out, const void* q_lat, long ql_t, long ql_h,
                                  const void* q_rot, long qr_t, long qr_h, const void* pages,
                                  const int* block_table, int bt_stride, const int* seq_of_token,
                                  const int* positions, int T, int heads, int rank, int rot,
                                  int page_size, float scale, int act_dt, cudaStream_t stream) {
  if (T <= 0) return HB_OK;
  if (heads <= 0 || rank <= 0 || rank > LA_MAX_RANK || rot < 0 || rank + rot > LA_MAX_ROW ||
      page_size <= 0)
    return HB_BAD_ARGUMENT;
  const int n_rows = T * heads;
  const int blocks = (n_rows + LA_WARPS - 1) / LA_WARPS;
  const size_t smem = (size_t)LA_WARPS * (rank + rot) * sizeof(float);
  HB_DISPATCH_DTYPE(act_dt, TA,
    hb_launch(latent_attention_kernel<TA>, dim3(blocks), dim3(LA_WARPS * 32), smem, stream,
              (TA*)out, (const TA*)q_lat, ql_t, ql_h, (const TA*)q_rot, qr_t, qr_h,
              (const TA*)pages, block_table, bt_stride, seq_of_token, positions, n_rows, heads,
              rank, rot, page_size, scale));
  return hb_check_launch();
}

// ---------------------------------------------------------------- attention on the tensor cores
// bfloat16, rank a multiple of 32 (at most 512), rot a multiple of 16.  All heads of all tokens
// of a request attend the same rows, so a block takes 32 query rows = (token, head) pairs of
// one request (`tokens_per_tile` tokens x `heads_per_block` heads) against tiles of 32 keys:
//
//   8 warps = 2 row groups of 16 rows x 4 column quarters.  Scores: warp (rg, cq) computes
//   the 16 x 8 block of its row group against keys 8 cq .. 8 cq + 7 (mma.sync m16n8k16 over
//   rank + rot), masks by position and leaves it in shared memory.  After a barrier every
//   warp of the row group does the online-softmax step (float32, base 2) for four of the 16
//   rows and leaves P (bfloat16) and the rows' rescale factors in shared memory; after a
//   second barrier every warp adds P V for its quarter of the latent's columns: V is the
//   first `rank` values of the very rows that were the keys, already in shared memory.
//
// Key tiles arrive by 16-byte cp.async, one tile ahead.  The keys of a request are cut into
// `n_splits` ranges (blockIdx.z), so that steps of few rows still fill the SMs; with more
// than one range the blocks leave unnormalised sums, maxima and weights, and
// `latent_attention_merge` puts them together.
#include "attention_mma.cuh"

constexpr int LM_ROWS = 32, LM_KEYS = 32, LM_MAXNT = 16, LM_SPAD = 36, LM_PPAD = 40;

// NTQ = rank / 32: the 8-column tiles of the latent a warp owns, a template parameter so that the
// loops over them unroll without predicates (with a run-time count, integer arithmetic and
// branches were most of the executed instructions and the tensor pipe a twentieth).
template <int NTQ>
__global__ void __launch_bounds__(256)
latent_attention_mma_kernel(__nv_bfloat16* __restrict__ out, float* __restrict__ part_acc,
                            float* __restrict__ part_ml,
                            const __nv_bfloat16* __restrict__ q_lat, long ql_t, long ql_h,
                            const __nv_bfloat16* __restrict__ q_rot, long qr_t, long qr_h,
                            const __nv_bfloat16* __restrict__ pages,
                            const int* __restrict__ block_table, int bt_stride,
                            const int* __restrict__ q_tiles, const int* __restrict__ cu_tokens,
                            const int* __restrict__ start_pos, int heads, int heads_per_block,
                            int tokens_per_tile, int rank, int rot, int page_size, int page_shift,
                            float scale_log2, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) unsigned char lm_smem[];
  const int D = rank + rot, RS = D + 8;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);      // [32][RS]
  __nv_bfloat16* k_s = q_s + LM_ROWS * RS;                             // [2][32][RS]
  float* s_s = reinterpret_cast<float*>(k_s + 2 * LM_KEYS * RS);       // [32][LM_SPAD]
  int* row_pos = reinterpret_cast<int*>(s_s + LM_ROWS * LM_SPAD);      // [32]
  int* row_out = row_pos + LM_ROWS;                                    // [32]: token * heads + head, -1 for none
  float* corr_s = reinterpret_cast<float*>(row_out + LM_ROWS);         // [32]
  float* m_s = corr_s + LM_ROWS;                                       // [32]
  float* l_s = m_s + LM_ROWS;                                          // [32]
  __nv_bfloat16* p_s = reinterpret_cast<__nv_bfloat16*>(l_s + LM_ROWS);  // [32][LM_PPAD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp >> 2, cq = warp & 3, g = lane >> 2, t4 = lane & 3;
  const int seq = q_tiles[2 * blockIdx.x], t_first = q_tiles[2 * blockIdx.x + 1];
  const int tok0 = cu_tokens[seq], n_tok = cu_tokens[seq + 1] - tok0;
  if (t_first >= n_tok) return;                       // a tile that holds no work
  const int h0 = blockIdx.y * heads_per_block;
  const int split = blockIdx.z;
  const int* table = block_table + (size_t)seq * bt_stride;
  const int last_tok = min(t_first + tokens_per_tile, n_tok);
  const int n_keys = start_pos[seq] + last_tok;       // the tile's last token sees this many keys
  const int n_kt = (n_keys + LM_KEYS - 1) / LM_KEYS;
  const int per = (n_kt + n_splits - 1) / n_splits;
  const int kt_lo = split * per, kt_hi = min(n_kt, kt_lo + per);

  if (tid < LM_ROWS) {
    const int lt = tid / heads_per_block, h = h0 + tid % heads_per_block;
    const bool ok = lt < tokens_per_tile && t_first + lt < n_tok && h < heads;
    row_pos[tid] = ok ? start_pos[seq] + t_first + lt : -1;
    row_out[tid] = ok ? (tok0 + t_first + lt) * heads + h : -1;
  }
  __syncthreads();
  // rows are handed out from 0 on: a group whose first row is none has none (steps of single
  // tokens with 16 heads or fewer fill one group only)
  const bool group_live = row_out[rg * 16] >= 0;
  // a warp copies 4 query rows (index arithmetic once a row, not once a value)
  for (int r = warp; r < LM_ROWS; r += 8) {
    __nv_bfloat16* dst = q_s + r * RS;
    if (row_out[r] >= 0) {
      const int tg = row_out[r] / heads, h = row_out[r] - tg * heads;
      const __nv_bfloat16* ql = q_lat + (size_t)tg * ql_t + (size_t)h * ql_h;
      const __nv_bfloat16* qr = q_rot + (size_t)tg * qr_t + (size_t)h * qr_h;
      for (int d = lane; d < rank; d += 32) dst[d] = ql[d];
      for (int d = lane; d < rot; d += 32) dst[rank + d] = qr[d];
    } else {
      for (int d = lane; d < D; d += 32) dst[d] = __float2bfloat16_rn(0.f);
    }
  }

  // Lane r finds the row of key kt * 32 + r (its page from the block table); warp w then
  // copies rows 4 w .. 4 w + 3 in 16-byte pieces, the row's start handed over by shuffles:
  // no division per piece.  Rows beyond the last key are zero-filled.
  const int vec_per_row = D / 8;
  auto load_tile = [&](int kt, int buf) {
    __nv_bfloat16* dst = k_s + (size_t)buf * LM_KEYS * RS;
    const int key = kt * LM_KEYS + lane;
    long long row_off = -1;
    if (key < n_keys) {
      const int pg = page_shift >= 0 ? key >> page_shift : key / page_size;
      const int in_pg = page_shift >= 0 ? key & (page_size - 1) : key - pg * page_size;
      row_off = ((long long)table[pg] * page_size + in_pg) * D;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = 4 * warp + i;
      const long long off = __shfl_sync(0xffffffffu, row_off, r);
      const __nv_bfloat16* src = pages + (off < 0 ? 0 : off);
      __nv_bfloat16* drow = dst + r * RS;
      for (int v = lane; v < vec_per_row; v += 32) cp_async16(drow + v * 8, src + v * 8, off < 0 ? 0 : 16);
    }
  };

  float acc[NTQ][4];
#pragma unroll
  for (int i = 0; i < NTQ; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
  float m_row = -INFINITY, l_row = 0.f;               // of row rg * 16 + 4 cq + lane / 8 (eight lanes hold a copy)
  const int col_q = cq * (rank / 4);
  const int ksteps = D / 16;

  if (kt_lo < kt_hi) load_tile(kt_lo, 0);
  cp_async_commit();
  int buf = 0;
  for (int kt = kt_lo; kt < kt_hi; ++kt) {
    cp_async_wait<0>();
    __syncthreads();
    if (kt + 1 < kt_hi) load_tile(kt + 1, buf ^ 1);
    cp_async_commit();
    const __nv_bfloat16* kt_s = k_s + (size_t)buf * LM_KEYS * RS;
    // scores of 16 rows against 8 keys (a row group without rows only keeps the barriers)
    if (group_live) {
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      const __nv_bfloat16* krow = kt_s + (8 * cq + g) * RS + 2 * t4;
      // one ldmatrix.x4 gives the key fragments of two k-steps: matrix j = columns 8 j .. 8 j + 7
      const __nv_bfloat16* kmat = kt_s + (8 * cq + (lane & 7)) * RS + (lane >> 3) * 8;
      const __nv_bfloat16* qbase = q_s + (rg * 16 + (lane & 15)) * RS + (lane >> 4) * 8;
      // two accumulators: two chains of dependent mma instead of one
      float c1[4] = {0.f, 0.f, 0.f, 0.f};
      int ks = 0;
      for (; ks + 1 < ksteps; ks += 2) {
        uint32_t a0[4], a1[4], b[4];
        ldmatrix_x4(a0, qbase + ks * 16);
        ldmatrix_x4(a1, qbase + ks * 16 + 16);
        ldmatrix_x4(b, kmat + ks * 16);
        mma_bf16(c, a0, b[0], b[1]);
        mma_bf16(c1, a1, b[2], b[3]);
      }
      if (ks < ksteps) {
        uint32_t a[4];
        ldmatrix_x4(a, qbase + ks * 16);
        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + ks * 16);
        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + ks * 16 + 8);
        mma_bf16(c, a, b0, b1);
      }
#pragma unroll
      for (int e = 0; e < 4; ++e) c[e] += c1[e];
      const int key = kt * LM_KEYS + 8 * cq + 2 * t4;
      const int ra = rg * 16 + g, rb = ra + 8;
      const int pa = row_pos[ra], pb = row_pos[rb];
      s_s[ra * LM_SPAD + 8 * cq + 2 * t4] = key <= pa ? c[0] * scale_log2 : -INFINITY;
      s_s[ra * LM_SPAD + 8 * cq + 2 * t4 + 1] = key + 1 <= pa ? c[1] * scale_log2 : -INFINITY;
      s_s[rb * LM_SPAD + 8 * cq + 2 * t4] = key <= pb ? c[2] * scale_log2 : -INFINITY;
      s_s[rb * LM_SPAD + 8 * cq + 2 * t4 + 1] = key + 1 <= pb ? c[3] * scale_log2 : -INFINITY;
    }
    __syncthreads();
    // online softmax, once a row: warp cq of a row group takes its rows 4 cq .. 4 cq + 3, eight
    // lanes a row with four keys each; P goes to shared memory as bfloat16, the factor by
    // which the row's earlier sums shrink beside it
    if (group_live) {
      const int row = rg * 16 + 4 * cq + (lane >> 3), c0 = (lane & 7) * 4;
      const float4 sv = *reinterpret_cast<const float4*>(s_s + row * LM_SPAD + c0);
      float mx = fmaxf(fmaxf(sv.x, sv.y), fmaxf(sv.z, sv.w));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
      const float m_new = fmaxf(m_row, mx);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
      const float corr = exp2f(m_row - m_use);
      m_row = m_new;
      const float p0 = exp2f(sv.x - m_use), p1 = exp2f(sv.y - m_use);
      const float p2 = exp2f(sv.z - m_use), p3 = exp2f(sv.w - m_use);
      float sum = (p0 + p1) + (p2 + p3);
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      l_row = l_row * corr + sum;
      uint2 packed;
      packed.x = pack_bf16(p0, p1);
      packed.y = pack_bf16(p2, p3);
      *reinterpret_cast<uint2*>(p_s + row * LM_PPAD + c0) = packed;
      if ((lane & 7) == 0) corr_s[row] = corr;
    }
    __syncthreads();
    if (!group_live) {
      buf ^= 1;
      continue;
    }
    // P V for this warp's quarter of the columns
    uint32_t pfrag[2][4];
    {
      const __nv_bfloat16* pbase = p_s + (rg * 16 + (lane & 15)) * LM_PPAD + (lane >> 4) * 8;
      ldmatrix_x4(pfrag[0], pbase);
      ldmatrix_x4(pfrag[1], pbase + 16);
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float corr = corr_s[rg * 16 + g + 8 * r];
        if (corr != 1.f) {                 // the maximum moved: rare once a row has seen a few tiles
#pragma unroll
          for (int nt = 0; nt < NTQ; ++nt) {
            acc[nt][2 * r] *= corr;
            acc[nt][2 * r + 1] *= corr;
          }
        }
      }
    }
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
      const __nv_bfloat16* vbase = kt_s + (16 * kk + ((lane >> 3) & 1) * 8 + (lane & 7)) * RS + col_q + (lane >> 4) * 8;
#pragma unroll
      for (int dp = 0; dp < (NTQ + 1) / 2; ++dp) {
        uint32_t r4[4];
        ldmatrix_x4_trans(r4, vbase + 16 * dp);
        mma_bf16(acc[2 * dp], pfrag[kk], r4[0], r4[1]);
        if (2 * dp + 1 < NTQ) mma_bf16(acc[2 * dp + 1], pfrag[kk], r4[2], r4[3]);
      }
    }
    buf ^= 1;
  }
  cp_async_wait<0>();
  if ((lane & 7) == 0) {
    m_s[rg * 16 + 4 * cq + (lane >> 3)] = m_row;
    l_s[rg * 16 + 4 * cq + (lane >> 3)] = l_row;
  }
  __syncthreads();
  float m[2], l[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    m[r] = m_s[rg * 16 + g + 8 * r];
    l[r] = l_s[rg * 16 + g + 8 * r];
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row_out[rg * 16 + g + 8 * r];
    if (row < 0) continue;
    if (n_splits == 1) {
      const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
      __nv_bfloat16* dst = out + (size_t)row * rank + col_q + 2 * t4;
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt)
        *reinterpret_cast<__nv_bfloat162*>(dst + 8 * nt) =
            __floats2bfloat162_rn(acc[nt][2 * r] * inv, acc[nt][2 * r + 1] * inv);
    } else {
      float* dst = part_acc + ((size_t)row * n_splits + split) * rank + col_q + 2 * t4;
#pragma unroll
      for (int nt = 0; nt < NTQ; ++nt)
        *reinterpret_cast<float2*>(dst + 8 * nt) = make_float2(acc[nt][2 * r], acc[nt][2 * r + 1]);
      if (cq == 0 && t4 == 0) {
        part_ml[((size_t)row * n_splits + split) * 2] = m[r];
        part_ml[((size_t)row * n_splits + split) * 2 + 1] = l[r];
      }
    }
  }
}

// out[row] = sum_i 2^(m_i - M) acc_i / sum_i 2^(m_i - M) l_i over the ranges, i in order
__global__ void latent_attention_merge_kernel(__nv_bfloat16* __restrict__ out,
                                              const float* __restrict__ part_acc,
                                              const float* __restrict__ part_ml, int n_rows,
                                              int rank, int n_splits) {
  pdl_launch_dependents();
  pdl_wait();
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  const float* ml = part_ml + (size_t)row * n_splits * 2;
  float M = -INFINITY;
  for (int i = 0; i < n_splits; ++i) M = fmaxf(M, ml[2 * i]);
  float L = 0.f;
  for (int i = 0; i < n_splits; ++i) L += (ml[2 * i] == -INFINITY ? 0.f : exp2f(ml[2 * i] - M)) * ml[2 * i + 1];
  const float inv = L > 0.f ? 1.f / L : 0.f;
  for (int d = lane; d < rank; d += 32) {
    float a = 0.f;
    for (int i = 0; i < n_splits; ++i) {
      const float w = ml[2 * i] == -INFINITY ? 0.f : exp2f(ml[2 * i] - M);
      a = fmaf(w, part_acc[((size_t)row * n_splits + i) * rank + d], a);
    }
    out[(size_t)row * rank + d] = __float2bfloat16_rn(a * inv);
  }
}

HB_EXPORT int hb_latent_attention_mma(void* out, float* part_acc, float* part_ml, const void* q_lat,
                                      long ql_t, long ql_h, const void* q_rot, long qr_t, long qr_h,
                                      const void* pages, const int* block_table, int bt_stride,
                                      const int* q_tiles, int n_tiles, const int* cu_tokens,
                                      const int* start_pos, int n_tokens, int heads,
                                      int heads_per_block, int tokens_per_tile, int rank, int rot,
                                      int page_size, float scale, int n_splits, cudaStream_t stream) {
  if (n_tiles <= 0 || n_tokens <= 0) return HB_OK;
  if (rank <= 0 || rank % 32 || rank > 32 * LM_MAXNT || rot < 0 || rot % 16 || heads <= 0 ||
      heads_per_block <= 0 || heads_per_block > LM_ROWS || tokens_per_tile <= 0 ||
      tokens_per_tile * heads_per_block > LM_ROWS || page_size <= 0 || n_splits <= 0 ||
      n_splits > 65535 || (n_splits > 1 && (part_acc == nullptr || part_ml == nullptr)))
    return HB_BAD_ARGUMENT;
  const int RS = rank + rot + 8;
  const size_t smem = (size_t)3 * LM_ROWS * RS * 2 + (size_t)LM_ROWS * LM_SPAD * 4 + 5 * LM_ROWS * 4 +
                      (size_t)LM_ROWS * LM_PPAD * 2;
  if (smem > 220 * 1024) return HB_BAD_ARGUMENT;
  const int head_groups = (heads + heads_per_block - 1) / heads_per_block;
  int page_shift = -1;                               // log2 of a page size that is a power of two
  for (int b = 0; b < 31; ++b)
    if ((1 << b) == page_size) page_shift = b;
  static size_t smem_set[LM_MAXNT + 1] = {};
#define HB_LM_LAUNCH(N)                                                                              \
  case N:                                                                                            \
    if (smem > 48 * 1024 && smem > smem_set[N]) {                                                    \
      if (cudaFuncSetAttribute(latent_attention_mma_kernel<N>,                                       \
                               cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
        return HB_LAUNCH_FAILED;                                                                     \
      smem_set[N] = smem;                                                                            \
    }                                                                                                \
    hb_launch(latent_attention_mma_kernel<N>, dim3(n_tiles, head_groups, n_splits), dim3(256), smem, \
              stream, (__nv_bfloat16*)out, part_acc, part_ml, (const __nv_bfloat16*)q_lat, ql_t, ql_h, \
              (const __nv_bfloat16*)q_rot, qr_t, qr_h, (const __nv_bfloat16*)pages, block_table,     \
              bt_stride, q_tiles, cu_tokens, start_pos, heads, heads_per_block, tokens_per_tile, rank, \
              rot, page_size, page_shift, scale * 1.4426950408889634f, n_splits);                    \
    break;
  switch (rank / 32) {
    HB_LM_LAUNCH(1) HB_LM_LAUNCH(2) HB_LM_LAUNCH(3) HB_LM_LAUNCH(4) HB_LM_LAUNCH(5) HB_LM_LAUNCH(6)
    HB_LM_LAUNCH(7) HB_LM_LAUNCH(8) HB_LM_LAUNCH(9) HB_LM_LAUNCH(10) HB_LM_LAUNCH(11) HB_LM_LAUNCH(12)
    HB_LM_LAUNCH(13) HB_LM_LAUNCH(14) HB_LM_LAUNCH(15) HB_LM_LAUNCH(16)
    default: return HB_BAD_ARGUMENT;
  }
#undef HB_LM_LAUNCH
  if (n_splits > 1) {
    const int n_rows = n_tokens * heads;
    hb_launch(latent_attention_merge_kernel, dim3((n_rows + 3) / 4), dim3(128), 0, stream,
              (__nv_bfloat16*)out, (const float*)part_acc, (const float*)part_ml, n_rows, rank, n_splits);
  }
  return hb_check_launch();
}
