// Grouped-query softmax attention over a sliding window of tokens and, before the window, one pooled key and value
// per block of P tokens.  A query at position i reads the tokens j with 0 <= i - j < window, and block b (the
// positions b P .. b P + P - 1) once the whole block lies before the window: b P + P - 1 <= i - window.  A pooled key
// is the mean of the block's keys as the pages hold them (after norm and rotation), a pooled value the mean of its
// values; tokens and blocks share one softmax.  Scores may be capped: s <- cap * tanh(s / cap).
//
// Two caches per layer run: pages with one entry per token (planes k [G, D] and v [G, Dv]), of which the manager
// keeps the last max(window, P) tokens' pages, and pages with one entry per block (planes pk and pv), kept for good.
//
//   pw_qkv_post      RMS norm of the whole q projection and of the whole k projection (one mean over all heads'
//                    values, a weight per value), rotation of the first `dims` values of every head (pair i with
//                    i + dims / 2, sines and cosines times `mag`), q to a buffer, k and v into the token pages
//   pool_blocks      the blocks that this step completed: their means into the block pages
//   pw_attn_ref      a warp per (token, head), blocks first and then tokens, one by one in ascending order, float32
//                    arithmetic: the float32 run's kernel, the fallback for every shape and the other kernels' oracle
// The bfloat16 run's kernel for heads of 32, 64 or 128 values (tensor cores) is in pooled_attn_mma.cu.
#include "common.cuh"

namespace q3 {

constexpr int PW_PER = 16;  // values per lane: head sizes up to 512

// proj: [T, ld]: q (H * D values) at column 0, k (G * D) at k_col, v (G * Dv) at v_col.
template <typename T>
__global__ void pw_qkv_post_kernel(const T* __restrict__ proj, int ld, int k_col, int v_col, int H, int G, int D, int Dv,
                                   const float* __restrict__ wq, const float* __restrict__ wk, float eps, int dims,
                                   const float* __restrict__ freq, float mag, const int* __restrict__ positions,
                                   const int* __restrict__ tok_seq, const int* __restrict__ table, int stride,
                                   int page_size, int num_pages, T* __restrict__ q_out, T* __restrict__ k_pages,
                                   T* __restrict__ v_pages, int write_cache, int* status) {
  extern __shared__ float cs[];  // [dims / 2] cosines, then [dims / 2] sines, times mag
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;
  const int pos = positions[t], b = tok_seq[t];
  const int half = dims >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, c;
    sincosf((float)pos * freq[i], &sn, &c);
    cs[i] = c * mag;
    cs[half + i] = sn * mag;
  }
  float ssq = 0.f, ssk = 0.f;
  for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
    const float v = to_float(row[i]);
    ssq = fmaf(v, v, ssq);
  }
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const float v = to_float(row[k_col + i]);
    ssk = fmaf(v, v, ssk);
  }
  // without norm weights (wq null) q and k pass as projected; block_sum's barriers also publish cs
  const float rq = wq ? 1.0f / sqrtf(block_sum(ssq, red) / (float)(H * D) + eps) : 1.0f;
  const float rk = wq ? 1.0f / sqrtf(block_sum(ssk, red) / (float)(G * D) + eps) : 1.0f;
  if (!wq) __syncthreads();
  for (int i = threadIdx.x; i < H * D; i += blockDim.x) {
    const int d = i % D;
    float v = wq ? to_float(row[i]) * rq * wq[i] : to_float(row[i]);
    if (d < dims) {
      const int p = d < half ? d : d - half;
      const int o = d < half ? i + half : i - half;
      const float u = wq ? to_float(row[o]) * rq * wq[o] : to_float(row[o]);
      v = d < half ? v * cs[p] - u * cs[half + p] : v * cs[p] + u * cs[half + p];
    }
    q_out[(size_t)t * H * D + i] = from_float<T>(v);
  }
  if (!write_cache) return;
  if (pos < 0 || b < 0) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int page = table_page(table + (size_t)b * stride, pos / page_size, stride, status);
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
    return;
  }
  const int in_page = pos % page_size;
  for (int i = threadIdx.x; i < G * D; i += blockDim.x) {
    const int g = i / D, d = i - g * D;
    float v = wk ? to_float(row[k_col + i]) * rk * wk[i] : to_float(row[k_col + i]);
    if (d < dims) {
      const int p = d < half ? d : d - half;
      const int o = d < half ? i + half : i - half;
      const float u = wk ? to_float(row[k_col + o]) * rk * wk[o] : to_float(row[k_col + o]);
      v = d < half ? v * cs[p] - u * cs[half + p] : v * cs[p] + u * cs[half + p];
    }
    k_pages[(((size_t)page * G + g) * page_size + in_page) * D + d] = from_float<T>(v);
  }
  for (int i = threadIdx.x; i < G * Dv; i += blockDim.x) {
    const int g = i / Dv, d = i - g * Dv;
    v_pages[(((size_t)page * G + g) * page_size + in_page) * Dv + d] = row[v_col + i];
  }
}

// Block (x, b): the x-th block of P tokens that request b completed in this step (its last token is one of the
// step's).  Sums ascending over the block's tokens in float32, then one division.
template <typename T>
__global__ void pool_blocks_kernel(const T* __restrict__ k_pages, const T* __restrict__ v_pages, T* __restrict__ pk_pages,
                                   T* __restrict__ pv_pages, const int* __restrict__ q_start, const int* __restrict__ kv_len,
                                   const int* __restrict__ table, int stride, int num_pages, const int* __restrict__ ptable,
                                   int pstride, int num_ppages, int page_size, int G, int D, int Dv, int P, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y;
  const int len = kv_len[b];
  const int start = len - (q_start[b + 1] - q_start[b]);
  if (start < 0) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int blk = start / P + blockIdx.x;
  if (blk >= len / P) return;
  const int ppage = table_page(ptable + (size_t)b * pstride, blk / page_size, pstride, status);
  if (ppage < 0 || ppage >= num_ppages) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
    return;
  }
  const int* row = table + (size_t)b * stride;
  const int p_in = blk % page_size;
  const float count = (float)P;
  // one value per thread; the block's tokens are asked for eight at a time, so that the loads overlap
  const int i = blockIdx.z * blockDim.x + threadIdx.x;
  if (i >= G * (D + Dv)) return;
  const bool is_k = i < G * D;
  const int e = is_k ? i : i - G * D;
  const int width = is_k ? D : Dv;
  const int g = e / width, d = e - g * width;
  const T* pages = is_k ? k_pages : v_pages;
  float sum = 0.f;
  bool bad = false;
  for (int j0 = 0; j0 < P; j0 += 8) {
    float part[8];
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const int pos = blk * P + min(j0 + jj, P - 1);
      int page = table_page(row, pos / page_size, stride, status);
      if (page < 0 || page >= num_pages) {
        bad = true;
        page = 0;
      }
      part[jj] = to_float(pages[(((size_t)page * G + g) * page_size + pos % page_size) * width + d]);
    }
#pragma unroll
    for (int jj = 0; jj < 8; ++jj)
      if (j0 + jj < P) sum += part[jj];
  }
  if (bad) {
    atomicOr(status, Q3_STATUS_BAD_PAGE);
    sum = 0.f;
  }
  T* dst = is_k ? pk_pages : pv_pages;
  dst[(((size_t)ppage * G + g) * page_size + p_in) * width + d] = from_float<T>(sum / count);
}

template <typename T>
__global__ void __launch_bounds__(128)
pw_attn_ref_kernel(const T* __restrict__ q, const T* __restrict__ k_pages, const T* __restrict__ v_pages,
                   const T* __restrict__ pk_pages, const T* __restrict__ pv_pages, const int* __restrict__ positions,
                   const int* __restrict__ tok_seq, const int* __restrict__ table, int stride, int num_pages,
                   const int* __restrict__ ptable, int pstride, int num_ppages, int page_size, T* __restrict__ out, int ldo,
                   int Ttot, int H, int G, int D, int Dv, int window, int P, float scale, float cap, float out_scale,
                   int block_limit, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (unit >= Ttot * H) return;
  const int t = unit / H, h = unit - t * H;
  const int g = h / (H / G);
  const int pos = positions[t], b = tok_seq[t];
  T* o = out + (size_t)t * ldo + (size_t)h * Dv;
  if (pos < 0 || b < 0) {
    if (lane == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    for (int d = lane; d < Dv; d += 32) o[d] = from_float<T>(0.f);
    return;
  }
  float qv[PW_PER], acc[PW_PER];
#pragma unroll
  for (int k = 0; k < PW_PER; ++k) {
    const int d = lane + 32 * k;
    qv[k] = d < D ? to_float(q[((size_t)t * H + h) * D + d]) : 0.f;
    acc[k] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int first = max(0, pos - window + 1);
  const int blocks = min(first / P, block_limit);  // the blocks that end before the window, the first so many of them
  const int* prow = ptable + (size_t)b * pstride;
  const int* row = table + (size_t)b * stride;
  const int total = blocks + (pos - first + 1);
  for (int n = 0; n < total; ++n) {
    const bool pooled = n < blocks;
    const int idx = pooled ? n : first + (n - blocks);
    const int page = pooled ? table_page(prow, idx / page_size, pstride, status)
                            : table_page(row, idx / page_size, stride, status);
    if (page < 0 || page >= (pooled ? num_ppages : num_pages)) {
      if (lane == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
      continue;
    }
    const size_t slot = ((size_t)page * G + g) * page_size + idx % page_size;
    const T* kv = (pooled ? pk_pages : k_pages) + slot * D;
    const T* vv = (pooled ? pv_pages : v_pages) + slot * Dv;
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < PW_PER; ++k) {
      const int d = lane + 32 * k;
      if (d < D) dot = fmaf(qv[k], to_float(kv[d]), dot);
    }
    float s = warp_sum(dot) * scale;
    if (cap > 0.f) s = cap * tanhf(s / cap);
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new), p = expf(s - m_new);  // m = -inf at the first key: corr = 0
    l = fmaf(l, corr, p);
#pragma unroll
    for (int k = 0; k < PW_PER; ++k) {
      const int d = lane + 32 * k;
      if (d < Dv) acc[k] = fmaf(acc[k], corr, p * to_float(vv[d]));
    }
    m = m_new;
  }
  const float inv = l > 0.f ? out_scale / l : 0.f;
#pragma unroll
  for (int k = 0; k < PW_PER; ++k) {
    const int d = lane + 32 * k;
    if (d < Dv) o[d] = from_float<T>(acc[k] * inv);
  }
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

extern "C" int q3_pw_qkv_post(const void* proj, int ld, int k_col, int v_col, int H, int G, int D, int Dv, const float* wq,
                              const float* wk, float eps, int dims, const float* freq, float mag, const int* positions,
                              const int* tok_seq, const int* table, int stride, int page_size, int num_pages, void* q_out,
                              void* k_pages, void* v_pages, int write_cache, int dtype, int T, int* status,
                              cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || Dv <= 0 || dims < 0 || dims > D || dims % 2 || dims > 8192 || page_size <= 0 ||
      stride <= 0)
    return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::pw_qkv_post_kernel<E>, dim3(T), dim3(256), (size_t)dims * sizeof(float), stream,
                                (const E*)proj, ld, k_col, v_col, H, G, D, Dv, wq, wk, eps, dims, freq, mag, positions,
                                tok_seq, table, stride, page_size, num_pages, (E*)q_out, (E*)k_pages, (E*)v_pages,
                                write_cache, status))
  return q3::launch_status();
}

// max_blocks: an upper bound of the blocks one request completes in this step (from its longest portion).
extern "C" int q3_pool_blocks(const void* k_pages, const void* v_pages, void* pk_pages, void* pv_pages, const int* q_start,
                              const int* kv_len, const int* table, int stride, int num_pages, const int* ptable,
                              int pstride, int num_ppages, int page_size, int G, int D, int Dv, int P, int B,
                              int max_blocks, int dtype, int* status, cudaStream_t stream) {
  if (B <= 0 || max_blocks <= 0) return 0;
  if (G <= 0 || D <= 0 || Dv <= 0 || P <= 0 || page_size <= 0 || stride <= 0 || pstride <= 0 || B > 65535) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::pool_blocks_kernel<E>, dim3(max_blocks, B, (G * (D + Dv) + 127) / 128), dim3(128), 0, stream, (const E*)k_pages,
                                (const E*)v_pages, (E*)pk_pages, (E*)pv_pages, q_start, kv_len, table, stride, num_pages,
                                ptable, pstride, num_ppages, page_size, G, D, Dv, P, status))
  return q3::launch_status();
}

// q: [T, H, D]; out: rows of `ldo` values, head h at column h * Dv, multiplied by out_scale.  cap <= 0: no cap.
// block_limit: only the first so many blocks are ever read (negative: all).  With P = 1 and the token pages given as
// the block pages too, that is a window that also keeps a request's first `block_limit` tokens.
extern "C" int q3_pw_attn_ref(const void* q, const void* k_pages, const void* v_pages, const void* pk_pages,
                              const void* pv_pages, const int* positions, const int* tok_seq, const int* table, int stride,
                              int num_pages, const int* ptable, int pstride, int num_ppages, int page_size, void* out,
                              int ldo, int dtype, int T, int H, int G, int D, int Dv, int window, int P, float scale,
                              float cap, float out_scale, int block_limit, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || D <= 0 || D > 32 * q3::PW_PER || Dv <= 0 || Dv > 32 * q3::PW_PER || window <= 0 ||
      P <= 0 || page_size <= 0 || stride <= 0 || pstride <= 0)
    return Q3_ERR_SIZE;
  const long long blocks = ((long long)T * H + 3) / 4;
  if (blocks > 0x7fffffffll) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::pw_attn_ref_kernel<E>, dim3((unsigned)blocks), dim3(128), 0, stream, (const E*)q,
                                (const E*)k_pages, (const E*)v_pages, (const E*)pk_pages, (const E*)pv_pages, positions,
                                tok_seq, table, stride, num_pages, ptable, pstride, num_ppages, page_size, (E*)out, ldo, T,
                                H, G, D, Dv, window, P, scale, cap, out_scale, block_limit < 0 ? 0x7fffffff : block_limit,
                                status))
  return q3::launch_status();
}
