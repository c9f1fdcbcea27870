// Attention through a latent: per token the cache holds one normed latent vector c (`rank` values) and one rotated
// key part r (`rot` values), shared by all heads.  A head's key is [W_uk,h c | r] and its value W_uv,h c, but neither
// is ever formed: with q' = W_uk,h^T q_plain the score is (q' . c + q_rot . r) * scale, and the head's output is
// W_uv,h (sum_j p_j c_j).  The kernels here do what lies around the matrix products:
//
//   latent_kv_post   norm of the query latent, norm of c and rotation of r into the pages, sigmoid of the output gates
//   latent_q_post    splits q into its plain part (packed for the product with W_uk) and its rotated part
//   latent_attn_ref  causal softmax attention over the pages, a warp per (token, head), keys one by one (float32
//                    arithmetic; the float32 run's kernel, every shape's fallback and the other kernels' oracle)
//   gate_heads       head outputs [H, T, dv] float32 times their gates -> [T, H dv] in the compute dtype
//
// Rotation: dimension i of the first `dims` of a rotated part is paired with i + dims / 2 (`pairing` 0, halves) or
// dimension 2i with 2i + 1 (`pairing` 1, neighbours); the angle is position * freq[i] in float32 and sine and cosine
// are multiplied by `mag` (the frequencies and the magnitude carry whatever stretching the model uses; the kernel
// only applies them).  A sink (`sink`, one logit per head, or null) takes part in the softmax's denominator only:
// weights exp(s_j) / (sum_j exp(s_j) + exp(sink_h)), with the scale on the scores s_j and not on the sink.
#include "common.cuh"

namespace q3 {

constexpr int LA_WARPS = 4;
constexpr int LA_PER = 16;      // latent values per lane: rank up to 512
constexpr int LA_ROT_PER = 4;   // rotated values per lane: rot up to 128

template <typename T>
__device__ __forceinline__ float rotated(const T* v, int i, int dims, const float* __restrict__ freq, float pos, float mag,
                                         int pairing) {
  // value i of the vector v after rotation; values from `dims` on pass unchanged
  if (i >= dims) return to_float(v[i]);
  const int half = dims >> 1;
  const int p = pairing ? i >> 1 : (i < half ? i : i - half);
  const bool first = pairing ? !(i & 1) : i < half;
  float s, c;
  sincosf(pos * freq[p], &s, &c);
  s *= mag;
  c *= mag;
  const float a = to_float(v[pairing ? 2 * p : p]), b = to_float(v[pairing ? 2 * p + 1 : p + half]);
  return first ? a * c - b * s : b * c + a * s;
}

// One block per token.  proj: [T, ld]: the query latent's pre-norm values at column 0 (q_rank of them), then the
// kv latent's (rank) and the shared key part (rot) from kv_col, then H gate pre-activations from gate_col.
template <typename T>
__global__ void latent_kv_post_kernel(const T* __restrict__ proj, int ld, int q_rank, int kv_col, int rank, int rot,
                                      int dims, int gate_col, int H, const float* __restrict__ wq,
                                      const float* __restrict__ wkv, float eps, const float* __restrict__ freq, float mag,
                                      const int* __restrict__ positions, const int* __restrict__ tok_seq,
                                      const int* __restrict__ table, int stride, int page_size, int num_pages,
                                      T* __restrict__ cq, T* __restrict__ c_pages, T* __restrict__ r_pages,
                                      float* __restrict__ gate, int write_cache, int pairing, int* status) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;
  float ssq = 0.f, ssk = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = to_float(row[i]);
    ssq = fmaf(v, v, ssq);
  }
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_float(row[kv_col + i]);
    ssk = fmaf(v, v, ssk);
  }
  const float rq = rsqrtf(block_sum(ssq, red) / (float)q_rank + eps);
  const float rk = rsqrtf(block_sum(ssk, red) / (float)rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[(size_t)t * q_rank + i] = from_float<T>(to_float(row[i]) * rq * wq[i]);
  if (gate)
    for (int h = threadIdx.x; h < H; h += blockDim.x)
      gate[(size_t)t * H + h] = sigmoid_f(to_float(row[gate_col + h]));
  if (!write_cache) return;
  const int pos = positions[t], b = tok_seq[t];
  if (pos < 0 || b < 0) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int page = table_page(table + (size_t)b * stride, pos / page_size, stride, status);
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
    return;
  }
  const size_t slot = (size_t)page * page_size + pos % page_size;
  for (int i = threadIdx.x; i < rank; i += blockDim.x)
    c_pages[slot * rank + i] = from_float<T>(to_float(row[kv_col + i]) * rk * wkv[i]);
  for (int i = threadIdx.x; i < rot; i += blockDim.x)
    r_pages[slot * rot + i] = from_float<T>(rotated(row + kv_col + rank, i, dims, freq, (float)pos, mag, pairing));
}

// One block per token.  q: [T, H, dn + rot] -> q_plain [T, H * dn] and q_rot [T, H, rot] (rotated).  The token's
// cosines and sines (dims / 2 of each, times mag) are worked out once per block.
template <typename T>
__global__ void latent_q_post_kernel(const T* __restrict__ q, int H, int dn, int rot, int dims,
                                     const float* __restrict__ freq, float mag, const int* __restrict__ positions,
                                     T* __restrict__ q_plain, T* __restrict__ q_rot, int pairing) {
  extern __shared__ float cs_table[];  // [dims / 2] cosines, then [dims / 2] sines
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int half = dims >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, c;
    sincosf(pos * freq[i], &sn, &c);
    cs_table[i] = c * mag;
    cs_table[half + i] = sn * mag;
  }
  __syncthreads();
  const int per = dn + rot;
  const T* row = q + (size_t)t * H * per;
  for (int i = threadIdx.x; i < H * per; i += blockDim.x) {
    const int h = i / per, d = i - h * per;
    if (d < dn) {
      q_plain[((size_t)t * H + h) * dn + d] = row[i];
      continue;
    }
    const int r = d - dn;
    const T* v = row + (size_t)h * per + dn;
    float out;
    if (r >= dims) {
      out = to_float(v[r]);
    } else {
      const int p = pairing ? r >> 1 : (r < half ? r : r - half);
      const bool first = pairing ? !(r & 1) : r < half;
      const float a = to_float(v[pairing ? 2 * p : p]), b = to_float(v[pairing ? 2 * p + 1 : p + half]);
      const float c = cs_table[p], sn = cs_table[half + p];
      out = first ? a * c - b * sn : b * c + a * sn;
    }
    q_rot[((size_t)t * H + h) * rot + r] = from_float<T>(out);
  }
}

// A warp per (token, head).  q_abs: float32 [H, T, rank]; q_rot: [T, H, rot]; pages of c [num_pages, page_size, rank]
// and of r [num_pages, page_size, rot]; out: [T, H * rank].  A token at position p reads the keys 0 .. p of its request.
template <typename T>
__global__ void __launch_bounds__(LA_WARPS * 32)
latent_attn_ref_kernel(const float* __restrict__ q_abs, const T* __restrict__ q_rot, const T* __restrict__ c_pages,
                       const T* __restrict__ r_pages, const int* __restrict__ positions, const int* __restrict__ tok_seq,
                       const int* __restrict__ table, int stride, int page_size, int num_pages, T* __restrict__ out,
                       int Ttot, int H, int rank, int rot, float scale, const float* __restrict__ sink, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * LA_WARPS + (threadIdx.x >> 5);
  if (unit >= Ttot * H) return;
  const int t = unit / H, h = unit - t * H;
  const int pos = positions[t], b = tok_seq[t];
  T* o = out + ((size_t)t * H + h) * rank;
  if (pos < 0 || b < 0) {
    if (lane == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    for (int r = lane; r < rank; r += 32) o[r] = from_float<T>(0.f);
    return;
  }
  float qa[LA_PER], acc[LA_PER], qr[LA_ROT_PER];
#pragma unroll
  for (int k = 0; k < LA_PER; ++k) {
    const int r = lane + 32 * k;
    qa[k] = r < rank ? q_abs[((size_t)h * Ttot + t) * rank + r] : 0.f;
    acc[k] = 0.f;
  }
#pragma unroll
  for (int k = 0; k < LA_ROT_PER; ++k) {
    const int r = lane + 32 * k;
    qr[k] = r < rot ? to_float(q_rot[((size_t)t * H + h) * rot + r]) : 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int* row = table + (size_t)b * stride;
  for (int j0 = 0; j0 <= pos; j0 += page_size) {
    const int page = table_page(row, j0 / page_size, stride, status);
    if (page < 0 || page >= num_pages) {
      if (lane == 0) atomicOr(status, Q3_STATUS_BAD_PAGE);
      continue;
    }
    const int n = min(page_size, pos + 1 - j0);
    for (int j = 0; j < n; ++j) {
      const size_t slot = (size_t)page * page_size + j;
      const T* cv = c_pages + slot * rank;
      const T* rv = r_pages + slot * rot;
      float c[LA_PER], dot = 0.f;
#pragma unroll
      for (int k = 0; k < LA_PER; ++k) {
        const int r = lane + 32 * k;
        c[k] = r < rank ? to_float(cv[r]) : 0.f;
        dot = fmaf(qa[k], c[k], dot);
      }
#pragma unroll
      for (int k = 0; k < LA_ROT_PER; ++k) {
        const int r = lane + 32 * k;
        if (r < rot) dot = fmaf(qr[k], to_float(rv[r]), dot);
      }
      const float s = warp_sum(dot) * scale;
      const float m_new = fmaxf(m, s);
      const float corr = expf(m - m_new), p = expf(s - m_new);  // m = -inf at the first key: corr = 0
      l = fmaf(l, corr, p);
#pragma unroll
      for (int k = 0; k < LA_PER; ++k) acc[k] = fmaf(acc[k], corr, p * c[k]);
      m = m_new;
    }
  }
  float keep = 1.f;
  if (sink) {  // one more term in the denominator, after the last key
    const float m_new = fmaxf(m, sink[h]);
    keep = expf(m - m_new);
    l = fmaf(l, keep, expf(sink[h] - m_new));
  }
  const float inv = l > 0.f ? keep / l : 0.f;
#pragma unroll
  for (int k = 0; k < LA_PER; ++k) {
    const int r = lane + 32 * k;
    if (r < rank) o[r] = from_float<T>(acc[k] * inv);
  }
}

// out[t, h * dv + v] = o[h, t, v] * gate[t, h] (without gates: the heads laid side by side)
template <typename T>
__global__ void gate_heads_kernel(const float* __restrict__ o, const float* __restrict__ gate, T* __restrict__ out,
                                  int Ttot, int H, int dv) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H * dv; i += blockDim.x) {
    const int h = i / dv, v = i - h * dv;
    out[(size_t)t * H * dv + i] = from_float<T>(o[((size_t)h * Ttot + t) * dv + v] * (gate ? gate[(size_t)t * H + h] : 1.f));
  }
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

extern "C" int q3_latent_kv_post(const void* proj, int ld, int q_rank, int kv_col, int rank, int rot, int dims, int gate_col,
                                 int H, const float* wq, const float* wkv, float eps, const float* freq, float mag,
                                 const int* positions, const int* tok_seq, const int* table, int stride, int page_size,
                                 int num_pages, void* cq, void* c_pages, void* r_pages, float* gate, int write_cache,
                                 int dtype, int T, int pairing, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (q_rank <= 0 || rank <= 0 || rot < 0 || dims < 0 || dims > rot || dims % 2 || H <= 0 || page_size <= 0 || stride <= 0)
    return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::latent_kv_post_kernel<E>, dim3(T), dim3(128), 0, stream, (const E*)proj, ld, q_rank,
                                kv_col, rank, rot, dims, gate_col, H, wq, wkv, eps, freq, mag, positions, tok_seq, table,
                                stride, page_size, num_pages, (E*)cq, (E*)c_pages, (E*)r_pages, gate, write_cache, pairing, status))
  return q3::launch_status();
}

extern "C" int q3_latent_q_post(const void* q, int H, int dn, int rot, int dims, const float* freq, float mag,
                                const int* positions, void* q_plain, void* q_rot, int dtype, int T, int pairing,
                                cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || dn <= 0 || rot < 0 || dims < 0 || dims > rot || dims % 2) return Q3_ERR_SIZE;
  if (dims > 8192) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::latent_q_post_kernel<E>, dim3(T), dim3(256), (size_t)dims * sizeof(float), stream,
                                (const E*)q, H, dn, rot, dims, freq, mag, positions, (E*)q_plain, (E*)q_rot, pairing))
  return q3::launch_status();
}

extern "C" int q3_latent_attn_ref(const float* q_abs, const void* q_rot, const void* c_pages, const void* r_pages,
                                  const int* positions, const int* tok_seq, const int* table, int stride, int page_size,
                                  int num_pages, void* out, int dtype, int T, int H, int rank, int rot, float scale,
                                  const float* sink, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || rank <= 0 || rank > 32 * q3::LA_PER || rot < 0 || rot > 32 * q3::LA_ROT_PER || page_size <= 0 || stride <= 0)
    return Q3_ERR_SIZE;
  const long long units = (long long)T * H;
  const long long blocks = (units + q3::LA_WARPS - 1) / q3::LA_WARPS;
  if (blocks > 0x7fffffffll) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::latent_attn_ref_kernel<E>, dim3((unsigned)blocks), dim3(q3::LA_WARPS * 32), 0, stream,
                                q_abs, (const E*)q_rot, (const E*)c_pages, (const E*)r_pages, positions, tok_seq, table,
                                stride, page_size, num_pages, (E*)out, T, H, rank, rot, scale, sink, status))
  return q3::launch_status();
}

extern "C" int q3_gate_heads(const float* o, const float* gate, void* out, int dtype, int T, int H, int dv,
                             cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || dv <= 0) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::gate_heads_kernel<E>, dim3(T), dim3(128), 0, stream, o, gate, (E*)out, T, H, dv))
  return q3::launch_status();
}
