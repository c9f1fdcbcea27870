// The matrix memory of the xLSTM (Beck et al., "xLSTM: Extended Long Short-Term Memory"), the mLSTM cell with
// exponential gates kept stable by a running maximum.  Per head: a memory S [D, Dv], a normaliser n [D] and the
// maximum m, all zero for a new request.  With q (already times D^-1/2), k [D], v [Dv] and the gates' pre-activations
// a_i, a_f of a token:
//
//   i = cap tanh((a_i + b_i) / cap)              f = logsigmoid(cap tanh((a_f + b_f) / cap))       (log gates)
//   m' = max(f + m, i);   S' = exp(f + m - m') S + exp(i - m') k v^T;   n' likewise with k alone
//   o = S'^T q / (max(|n' . q|, exp(-m')) + 1e-6)
//
//   mlstm_scan   walks the tokens of every request in order.  A block owns one head of one request and a slice of the
//                Dv columns; R lanes share a column and hold D / R values of it in registers; a chunk of tokens' q, k,
//                v and gates is staged in shared memory at a time.  The state is read at the start and written at
//                the end, so a prompt in portions walks exactly as the whole prompt does.
//   mlstm_out    each head's o divided by its root mean square, times a weight per value, times sigmoid of a gate
//                read from the mixer's input, times a scale: the operand of the output projection.
//
// Gates, decays, the state, n . q and the division are float32 in every run; q, k, v come as the projection left them.
#include "common.cuh"

namespace q3 {

constexpr int ML_THREADS = 128;
constexpr int ML_PER = 32;  // values of a column per lane

__device__ __forceinline__ float log_sigmoid_f(float x) { return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x)); }

template <typename T, int R>
__global__ void __launch_bounds__(ML_THREADS)
mlstm_scan_kernel(const T* __restrict__ proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                  const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                  float* __restrict__ S_state, float* __restrict__ n_state, float* __restrict__ m_state,
                  const int* __restrict__ q_start, const int* __restrict__ slot_ids, int num_slots, float* __restrict__ out,
                  int H, int D, int Dv, int chunk, int* status) {
  constexpr int COLS = ML_THREADS / R;
  extern __shared__ float ml_smem[];
  float* q_s = ml_smem;                    // [chunk][D]
  float* k_s = q_s + (size_t)chunk * D;    // [chunk][D]
  float* v_s = k_s + (size_t)chunk * D;    // [chunk][COLS]
  float* gi_s = v_s + (size_t)chunk * COLS;  // [chunk]
  float* gf_s = gi_s + chunk;               // [chunk]
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.z, h = blockIdx.y;
  const int col0 = blockIdx.x * COLS;
  const int slot = slot_ids[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int t0 = q_start[b], t1 = q_start[b + 1];
  const int r = threadIdx.x % R, lc = threadIdx.x / R;
  const int col = col0 + lc;
  const bool live = col < Dv;
  float* S_h = S_state + ((size_t)slot * H + h) * D * Dv;
  float* n_h = n_state + ((size_t)slot * H + h) * D;
  float S[ML_PER], n[ML_PER];
#pragma unroll
  for (int j = 0; j < ML_PER; ++j) {
    const int d = r + R * j;
    S[j] = (live && d < D) ? S_h[(size_t)d * Dv + col] : 0.f;
    n[j] = d < D ? n_h[d] : 0.f;
  }
  float m = m_state[(size_t)slot * H + h];
  const float bi = i_bias[h], bf = f_bias[h];
  for (int c0 = t0; c0 < t1; c0 += chunk) {
    const int cn = min(chunk, t1 - c0);
    __syncthreads();  // the chunk before has been walked by everybody
    for (int idx = threadIdx.x; idx < cn * D; idx += ML_THREADS) {
      const int c = idx / D, d = idx - c * D;
      const T* row = proj + (size_t)(c0 + c) * ld;
      q_s[c * D + d] = to_float(row[q_col + h * D + d]) * q_scale;
      k_s[c * D + d] = to_float(row[k_col + h * D + d]);
    }
    for (int idx = threadIdx.x; idx < cn * COLS; idx += ML_THREADS) {
      const int c = idx / COLS, j = idx - c * COLS;
      v_s[idx] = col0 + j < Dv ? to_float(proj[(size_t)(c0 + c) * ld + v_col + h * Dv + col0 + j]) : 0.f;
    }
    for (int c = threadIdx.x; c < cn; c += ML_THREADS) {
      const T* row = proj + (size_t)(c0 + c) * ld;
      gi_s[c] = cap * tanhf((to_float(row[i_col + h]) + bi) / cap);
      gf_s[c] = log_sigmoid_f(cap * tanhf((to_float(row[f_col + h]) + bf) / cap));
    }
    __syncthreads();
    for (int c = 0; c < cn; ++c) {
      const float gi = gi_s[c], gf = gf_s[c];
      const float m_new = fmaxf(gf + m, gi);
      const float keep = expf(gf + m - m_new), take = expf(gi - m_new);
      m = m_new;
      const float tv = take * v_s[c * COLS + lc];
      const float* kc = k_s + c * D;
      const float* qc = q_s + c * D;
      float num = 0.f, nq = 0.f;
#pragma unroll
      for (int j = 0; j < ML_PER; ++j) {
        const int d = r + R * j;
        if (d < D) {
          const float kd = kc[d], qd = qc[d];
          S[j] = fmaf(keep, S[j], tv * kd);
          n[j] = fmaf(keep, n[j], take * kd);
          num = fmaf(S[j], qd, num);
          nq = fmaf(n[j], qd, nq);
        }
      }
#pragma unroll
      for (int o = R >> 1; o > 0; o >>= 1) {  // the R lanes of a column are neighbours in a warp
        num += __shfl_xor_sync(0xffffffffu, num, o);
        nq += __shfl_xor_sync(0xffffffffu, nq, o);
      }
      if (live && r == 0) out[(size_t)(c0 + c) * H * Dv + (size_t)h * Dv + col] = num / (fmaxf(fabsf(nq), expf(-m)) + 1e-6f);
    }
  }
#pragma unroll
  for (int j = 0; j < ML_PER; ++j) {
    const int d = r + R * j;
    if (live && d < D) S_h[(size_t)d * Dv + col] = S[j];
    if (blockIdx.x == 0 && lc == 0 && d < D) n_h[d] = n[j];
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) m_state[(size_t)slot * H + h] = m;
}

// A warp per (token, head).  o: float32 [T, H * Dv]; the gates' pre-activations in proj [T, ld] from g_col; out: rows of
// `ldo` values in the compute dtype.
template <typename T>
__global__ void mlstm_out_kernel(const float* __restrict__ o, const T* __restrict__ proj, int ld, int g_col,
                                 const float* __restrict__ w, float eps, float out_scale, T* __restrict__ out, int ldo,
                                 int Ttot, int H, int Dv) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int unit = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= Ttot * H) return;
  const int t = unit / H, h = unit - t * H;
  const float* row = o + ((size_t)t * H + h) * Dv;
  float ss = 0.f;
  for (int v = lane; v < Dv; v += 32) ss = fmaf(row[v], row[v], ss);
  const float inv = out_scale / sqrtf(warp_sum(ss) / (float)Dv + eps);
  for (int v = lane; v < Dv; v += 32) {
    const float g = sigmoid_f(to_float(proj[(size_t)t * ld + g_col + h * Dv + v]));
    out[(size_t)t * ldo + h * Dv + v] = from_float<T>(row[v] * inv * w[h * Dv + v] * g);
  }
}

template <typename T, int R>
static int mlstm_scan_launch(const void* proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                             const float* i_bias, const float* f_bias, float cap, float* S, float* n, float* m,
                             const int* q_start, const int* slot_ids, int num_slots, float* out, int B, int H, int D, int Dv,
                             int* status, cudaStream_t stream) {
  constexpr int COLS = ML_THREADS / R;
  const int chunk = D > 256 ? 8 : 16;
  const size_t smem = ((size_t)chunk * (2 * D + COLS) + 2 * chunk) * sizeof(float);
  launch(mlstm_scan_kernel<T, R>, dim3((Dv + COLS - 1) / COLS, H, B), dim3(ML_THREADS), smem, stream, (const T*)proj, ld,
         q_col, k_col, v_col, i_col, f_col, i_bias, f_bias, cap, 1.0f / sqrtf((float)D), S, n, m, q_start, slot_ids,
         num_slots, out, H, D, Dv, chunk, status);
  return launch_status();
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

// The largest key size the scan takes.
extern "C" int q3_mlstm_max_dim() { return 16 * q3::ML_PER; }

// proj: [T, ld] in `dtype` with q and k (H * D each), v (H * Dv) and the gates' pre-activations (H each) at the given
// columns; i_bias, f_bias: float32 [H]; S [slots, H, D, Dv], n [slots, H, D], m [slots, H]: float32 state; out:
// float32 [T, H * Dv].  q is multiplied by D^-1/2.
extern "C" int q3_mlstm_scan(const void* proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                             const float* i_bias, const float* f_bias, float cap, float* S, float* n, float* m,
                             const int* q_start, const int* slot_ids, int num_slots, float* out, int dtype, int B, int H,
                             int D, int Dv, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || H > 65535 || B > 65535 || D <= 0 || D > 16 * q3::ML_PER || Dv <= 0 || cap <= 0.f || num_slots <= 0)
    return Q3_ERR_SIZE;
#define Q3_ML(R)                                                                                                       \
  Q3_BY_DTYPE(dtype, return (q3::mlstm_scan_launch<E, R>(proj, ld, q_col, k_col, v_col, i_col, f_col, i_bias, f_bias, cap, \
                                                         S, n, m, q_start, slot_ids, num_slots, out, B, H, D, Dv, status,  \
                                                         stream)))
  if (D <= q3::ML_PER) { Q3_ML(1) }
  if (D <= 2 * q3::ML_PER) { Q3_ML(2) }
  if (D <= 4 * q3::ML_PER) { Q3_ML(4) }
  if (D <= 8 * q3::ML_PER) { Q3_ML(8) }
  Q3_ML(16)
#undef Q3_ML
}

extern "C" int q3_mlstm_out(const float* o, const void* proj, int ld, int g_col, const float* w, float eps, float out_scale,
                            void* out, int ldo, int dtype, int T, int H, int Dv, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (H <= 0 || Dv <= 0 || ldo < H * Dv) return Q3_ERR_SIZE;
  const long long blocks = ((long long)T * H + 3) / 4;
  if (blocks > 0x7fffffffll) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::mlstm_out_kernel<E>, dim3((unsigned)blocks), dim3(128), 0, stream, o, (const E*)proj, ld,
                                g_col, w, eps, out_scale, (E*)out, ldo, T, H, Dv))
  return q3::launch_status();
}
