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
//                Dv columns; a warp owns a few columns, its lanes the rows of each, in registers; a chunk of tokens' q,
//                k, v and gates is staged in shared memory at a time, the next chunk fetched into registers meanwhile.
//                The state is read at the start and written at the end, so a prompt in portions walks exactly as the
//                whole prompt does.
//   segmented    (bfloat16, long portions) every request's portion is cut into segments of `seg` tokens that are walked
//                side by side: `mlstm_segments` lists them; the walk in its "local" mode takes every segment from an
//                empty memory to the memory, normaliser and maximum that the segment alone leaves, with the sum F of its
//                log forget gates; `mlstm_carry` goes through a request's segments in order, element by element:
//                entering with (S, m), a segment leaves  m' = max(F + m, m_loc),
//                S' = e^(F + m - m') S + e^(m_loc - m') S_loc  (which is the recurrence unrolled over the segment),
//                and what each segment enters with is kept; the walk in its "final" mode starts every segment from
//                that and writes the outputs, the last segment of a request also the request's state.  The sums are
//                the walk's in another order: results differ from the single walk by float32 rounding.
//   mlstm_out    each head's o divided by its root mean square, times a weight per value, times sigmoid of a gate
//                read from the mixer's input, times a scale: the operand of the output projection.
//
// Gates, decays, the state, n . q and the division are float32 in every run; q, k, v come as the projection left them.
#include "common.cuh"

namespace q3 {

constexpr int ML_WARPS = 4;
constexpr int ML_THREADS = 32 * ML_WARPS;
constexpr int ML_STAGE = 8;  // q and k values of a chunk that a thread fetches ahead

__device__ __forceinline__ float log_sigmoid_f(float x) { return x >= 0.f ? -log1pf(expf(-x)) : x - log1pf(expf(x)); }

// Sums of CPT values over the 32 lanes of a warp in log2(CPT) halving rounds and plain rounds after them: in a halving
// round a lane keeps the half of its values that its lane bit names and adds the partner's same half.  At the end
// v[0] of lane l is the total of value `warp_column<CPT>(l)`, the same in the lanes that differ in the low bits only.
// The order of the additions is fixed.
template <int CPT>
__device__ __forceinline__ void warp_sum_columns(float (&v)[CPT], int lane) {
  int width = CPT;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    if (width > 1) {
      const bool upper = lane & o;
      width >>= 1;
#pragma unroll
      for (int i = 0; i < CPT / 2; ++i) {
        if (i < width) {
          const float keep = upper ? v[i + width] : v[i], send = upper ? v[i] : v[i + width];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
      }
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
    }
  }
}
template <int CPT>
__device__ __forceinline__ int warp_column(int lane) {  // which of the CPT values a lane holds after warp_sum_columns
  int col = 0, width = CPT;
#pragma unroll
  for (int o = 16; o > 0 && width > 1; o >>= 1) {
    width >>= 1;
    if (lane & o) col += width;
  }
  return col;
}

// A warp owns CPT columns of S; lane l holds rows d = l + 32 j (j < PER) of each.  The memory is kept column by column,
// [slots, H, Dv, D], so that a warp reads and writes a column as runs of consecutive floats.  A chunk of CHUNK tokens
// is staged in shared memory (q times its scale, k, the block's columns of v, the log gates, and from them the
// chain of maxima and the three exponentials of every token); the next chunk is on its way into registers meanwhile.
// What a segment is: tokens t0 .. t1 - 1 of request `req`; `last`: the request's portion ends with it.
struct MlstmSegment {
  int t0, t1, req, last;
};
// Scratch of the segmented form, per segment: the memory it leaves alone and then the memory it starts from
// [segments, H, Dv, D], the normaliser likewise [segments, H, D], and [segments, H] each: the maximum it leaves alone,
// the sum of its log forget gates, the maximum it starts from.
struct MlstmScratch {
  float *S, *n, *m_loc, *F, *m_in;
};
constexpr int ML_PLAIN = 0, ML_LOCAL = 1, ML_FINAL = 2;

// One block: request b's portion becomes ceil(len / seg) segments, in the order of the requests.
__global__ void mlstm_segments_kernel(const int* __restrict__ q_start, int B, int seg, MlstmSegment* __restrict__ segments,
                                      int* __restrict__ first_of, int max_segments) {
  __shared__ int first[1025];
  pdl_wait();
  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    int at = 0;
    for (int b = 0; b < B; ++b) {
      first[b] = at;
      at += (q_start[b + 1] - q_start[b] + seg - 1) / seg;
    }
    first[B] = at;
  }
  __syncthreads();
  for (int b = threadIdx.x; b <= B; b += blockDim.x) first_of[b] = min(first[b], max_segments);
  for (int b = 0; b < B; ++b) {
    const int count = first[b + 1] - first[b], t0 = q_start[b], t1 = q_start[b + 1];
    for (int g = threadIdx.x; g < count; g += blockDim.x)
      if (first[b] + g < max_segments)
        segments[first[b] + g] = MlstmSegment{t0 + g * seg, min(t1, t0 + (g + 1) * seg), b, g == count - 1 ? 1 : 0};
  }
}

// grid (ceil(D * Dv / 256), H, B): element e of a request's memory (and, for e < D, of its normaliser) through the
// request's segments in order.
__global__ void mlstm_carry_kernel(const int* __restrict__ first_of, const int* __restrict__ slot_ids, int num_slots,
                                   const float* __restrict__ S_state, const float* __restrict__ n_state,
                                   const float* __restrict__ m_state, MlstmScratch scr, int H, int D, int Dv) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.z, h = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const int slot = slot_ids[b];
  if (slot < 0 || slot >= num_slots || e >= D * Dv) return;
  const size_t per = (size_t)D * Dv;
  float S = S_state[((size_t)slot * H + h) * per + e];
  float n = e < D ? n_state[((size_t)slot * H + h) * D + e] : 0.f;
  float m = m_state[(size_t)slot * H + h];
  for (int g = first_of[b]; g < first_of[b + 1]; ++g) {
    const size_t gh = (size_t)g * H + h;
    const float S_loc = scr.S[gh * per + e], m_loc = scr.m_loc[gh], F = scr.F[gh];
    scr.S[gh * per + e] = S;  // what the segment starts from
    const float m_new = fmaxf(F + m, m_loc);
    const float keep = expf(F + m - m_new), take = expf(m_loc - m_new);
    S = fmaf(keep, S, take * S_loc);
    if (e < D) {
      const float n_loc = scr.n[gh * D + e];
      scr.n[gh * D + e] = n;
      n = fmaf(keep, n, take * n_loc);
    }
    if (e == 0) scr.m_in[gh] = m;
    m = m_new;
  }
}

template <typename T, int PER, int CPT, int CHUNK, int MODE>
// the segments' walks at four blocks to an SM (128 registers: a long prompt's segments then run in two rounds instead of
// three); the single walk, bound by the latency of its own chain, keeps the registers it wants
__global__ void __launch_bounds__(ML_THREADS, MODE == ML_PLAIN ? 1 : 4)
mlstm_scan_kernel(const T* __restrict__ proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                  const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap, float q_scale,
                  float* __restrict__ S_state, float* __restrict__ n_state, float* __restrict__ m_state,
                  const int* __restrict__ q_start, const int* __restrict__ slot_ids, int num_slots, float* __restrict__ out,
                  int H, int D, int Dv, const MlstmSegment* __restrict__ segments, const int* __restrict__ first_of,
                  int num_requests, MlstmScratch scr, int* status) {
  constexpr int COLS = ML_WARPS * CPT;  // columns of a block
  constexpr int DP = 32 * PER;          // a row of q or k in shared memory: D values and zeros up to the lanes' reach
  constexpr int QK_STAGE = CHUNK * ((DP + ML_THREADS - 1) / ML_THREADS);
  constexpr int V_STAGE = (CHUNK * COLS + ML_THREADS - 1) / ML_THREADS;
  static_assert(QK_STAGE <= ML_STAGE, "a chunk that the threads can fetch ahead");
  __shared__ float q_s[CHUNK * DP], k_s[CHUNK * DP], v_s[CHUNK * COLS];
  __shared__ float gate_s[5 * CHUNK];  // log input gate, log forget gate; then keep, take, floor
  __shared__ float m_s[CHUNK + 1];
  pdl_wait();
  pdl_launch_dependents();
  // blockIdx.z: a request (plain mode) or a segment of the list (the other two)
  const int h = blockIdx.y;
  const int col0 = blockIdx.x * COLS;
  int b = blockIdx.z, t0, t1;
  bool writes_state = true;
  if (MODE == ML_PLAIN) {
    t0 = q_start[b], t1 = q_start[b + 1];
  } else {
    if ((int)blockIdx.z >= first_of[num_requests]) return;
    const MlstmSegment sg = segments[blockIdx.z];
    t0 = sg.t0, t1 = sg.t1, b = sg.req;
    writes_state = sg.last != 0;
  }
  const int slot = slot_ids[b];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wcol = col0 + warp * CPT;  // the warp's first column
  float* S_h = S_state + ((size_t)slot * H + h) * Dv * D;  // the request's own state
  float* n_h = n_state + ((size_t)slot * H + h) * D;
  const size_t gh = (size_t)blockIdx.z * H + h;            // the segment's scratch
  float S[CPT][PER], n[PER];
  {
    const float* S_from = MODE == ML_PLAIN ? S_h : scr.S + gh * Dv * D;
    const float* n_from = MODE == ML_PLAIN ? n_h : scr.n + gh * D;
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      const int d = lane + 32 * j;
      n[j] = (MODE != ML_LOCAL && d < D) ? n_from[d] : 0.f;
#pragma unroll
      for (int c = 0; c < CPT; ++c)
        S[c][j] = (MODE != ML_LOCAL && d < D && wcol + c < Dv) ? S_from[(size_t)(wcol + c) * D + d] : 0.f;
    }
  }
  // a segment alone starts from an empty memory: a maximum of minus infinity lets the first token's own gate in
  if (threadIdx.x == 0)
    m_s[0] = MODE == ML_PLAIN ? m_state[(size_t)slot * H + h] : (MODE == ML_LOCAL ? -INFINITY : scr.m_in[gh]);
  float F_sum = 0.f;  // thread 0, local mode: the segment's log forget gates added up
  const float bi = i_bias[h], bf = f_bias[h];

  // what a thread fetches of a chunk: ML_STAGE values of q and of k, V_STAGE of v, one token's gates
  T rq[QK_STAGE], rk[QK_STAGE], rv[V_STAGE], ri, rf;
  auto fetch = [&](int c0) {
    const int cn = min(CHUNK, t1 - c0);
#pragma unroll
    for (int i = 0; i < QK_STAGE; ++i) {  // token i % CHUNK, rows threadIdx.x + 128 * (i / CHUNK)
      const int c = i % CHUNK, d = threadIdx.x + (i / CHUNK) * ML_THREADS;
      const bool ok = c < cn && d < D;
      const T* row = proj + (size_t)(c0 + c) * ld + h * D + d;
      rq[i] = ok ? row[q_col] : from_float<T>(0.f);
      rk[i] = ok ? row[k_col] : from_float<T>(0.f);
    }
#pragma unroll
    for (int i = 0; i < V_STAGE; ++i) {
      const int idx = threadIdx.x + i * ML_THREADS;
      if (idx < cn * COLS) {
        const int c = idx / COLS, j = idx - c * COLS;
        rv[i] = col0 + j < Dv ? proj[(size_t)(c0 + c) * ld + v_col + h * Dv + col0 + j] : from_float<T>(0.f);
      }
    }
    if ((int)threadIdx.x < cn) {
      const T* row = proj + (size_t)(c0 + threadIdx.x) * ld;
      ri = row[i_col + h];
      rf = row[f_col + h];
    }
  };

  if (t0 < t1) fetch(t0);
  for (int c0 = t0; c0 < t1; c0 += CHUNK) {
    const int cn = min(CHUNK, t1 - c0);
    __syncthreads();  // the chunk before has been walked by everybody
#pragma unroll
    for (int i = 0; i < QK_STAGE; ++i) {
      const int c = i % CHUNK, d = threadIdx.x + (i / CHUNK) * ML_THREADS;
      if (d < DP) {  // zeros beyond D and beyond the chunk's tokens
        q_s[c * DP + d] = to_float(rq[i]) * q_scale;
        k_s[c * DP + d] = to_float(rk[i]);
      }
    }
#pragma unroll
    for (int i = 0; i < V_STAGE; ++i) {
      const int idx = threadIdx.x + i * ML_THREADS;
      if (idx < CHUNK * COLS) v_s[idx] = idx < cn * COLS ? to_float(rv[i]) : 0.f;
    }
    if ((int)threadIdx.x < cn) {
      gate_s[threadIdx.x] = cap * tanhf((to_float(ri) + bi) / cap);
      gate_s[CHUNK + threadIdx.x] = log_sigmoid_f(cap * tanhf((to_float(rf) + bf) / cap));
    }
    __syncthreads();
    if (c0 + CHUNK < t1) fetch(c0 + CHUNK);  // on its way while this chunk is walked
    if (threadIdx.x == 0) {  // the maxima are the one chain from token to token: m' = max(f + m, i)
      float gi[CHUNK], gf[CHUNK];
#pragma unroll
      for (int c = 0; c < CHUNK; ++c) gi[c] = gate_s[c], gf[c] = gate_s[CHUNK + c];
      float m = m_s[0];
#pragma unroll
      for (int c = 0; c < CHUNK; ++c) {
        if (c < cn) {
          m = fmaxf(gf[c] + m, gi[c]);
          if (MODE == ML_LOCAL) F_sum += gf[c];
        }
        m_s[c + 1] = m;
      }
    }
    __syncthreads();
    if ((int)threadIdx.x < CHUNK) {
      const int c = threadIdx.x;
      const float m_old = m_s[c], m_new = m_s[c + 1];
      const bool real = c < cn;  // a token beyond the chunk's end leaves the memory as it is
      gate_s[2 * CHUNK + c] = real ? expf(gate_s[CHUNK + c] + m_old - m_new) : 1.f;  // what stays of the memory
      gate_s[3 * CHUNK + c] = real ? expf(gate_s[c] - m_new) : 0.f;                   // what the token adds
      gate_s[4 * CHUNK + c] = expf(-m_new);                                            // the denominator's floor
    }
    __syncthreads();
    float num[CHUNK][CPT], nq[CHUNK];
#pragma unroll
    for (int c = 0; c < CHUNK; ++c) {
      nq[c] = 0.f;
#pragma unroll
      for (int i = 0; i < CPT; ++i) num[c][i] = 0.f;
    }
    // the memory's chain is one multiply-add per token and value; everything else of a token is independent of the
    // other tokens, and the loops are unrolled so that it overlaps
    // (no branches in here: rows beyond D and tokens beyond the chunk's end are zeros that change nothing)
#pragma unroll
    for (int c = 0; c < CHUNK; ++c) {
      const float keep = gate_s[2 * CHUNK + c], take = gate_s[3 * CHUNK + c];
      float vc[CPT];
#pragma unroll
      for (int i = 0; i < CPT; ++i) vc[i] = v_s[c * COLS + warp * CPT + i];
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int d = lane + 32 * j;
        const float kd = k_s[c * DP + d], qd = MODE == ML_LOCAL ? 0.f : q_s[c * DP + d];
        const float tk = take * kd;
        n[j] = fmaf(keep, n[j], tk);
        if (MODE != ML_LOCAL) nq[c] = fmaf(n[j], qd, nq[c]);  // a segment alone writes no outputs
        // two columns per instruction (the packed float32 multiply-add of sm_100): the same roundings as one by one
        const float2 keep2 = make_float2(keep, keep), tk2 = make_float2(tk, tk), qd2 = make_float2(qd, qd);
#pragma unroll
        for (int i = 0; i < CPT; i += 2) {
          float2 s2 = make_float2(S[i][j], S[i + 1][j]);
          s2 = __ffma2_rn(keep2, s2, __fmul2_rn(tk2, make_float2(vc[i], vc[i + 1])));
          S[i][j] = s2.x, S[i + 1][j] = s2.y;
          if (MODE != ML_LOCAL) {
            const float2 n2 = __ffma2_rn(s2, qd2, make_float2(num[c][i], num[c][i + 1]));
            num[c][i] = n2.x, num[c][i + 1] = n2.y;
          }
        }
      }
    }
    const int mine = warp_column<CPT>(lane);
#pragma unroll
    for (int c = 0; c < CHUNK; ++c) {
      if (MODE != ML_LOCAL && c < cn) {
        warp_sum_columns<CPT>(num[c], lane);
        float total = nq[c];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
        const int col = wcol + mine;
        if ((lane & (32 / CPT - 1)) == 0 && col < Dv)
          out[(size_t)(c0 + c) * H * Dv + (size_t)h * Dv + col] =
              num[c][0] / (fmaxf(fabsf(total), gate_s[4 * CHUNK + c]) + 1e-6f);
      }
    }
    if (threadIdx.x == 0) m_s[0] = m_s[cn];  // read again only after the next barrier
  }
  __syncthreads();
  if (MODE == ML_FINAL && !writes_state) return;  // only a request's last segment leaves the request's state
  float* S_to = MODE == ML_LOCAL ? scr.S + gh * Dv * D : S_h;
  float* n_to = MODE == ML_LOCAL ? scr.n + gh * D : n_h;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int d = lane + 32 * j;
    if (d >= D) continue;
    if (blockIdx.x == 0 && warp == 0) n_to[d] = n[j];
#pragma unroll
    for (int c = 0; c < CPT; ++c)
      if (wcol + c < Dv) S_to[(size_t)(wcol + c) * D + d] = S[c][j];
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (MODE == ML_LOCAL) {
      scr.m_loc[gh] = m_s[0];
      scr.F[gh] = F_sum;
    } else {
      m_state[(size_t)slot * H + h] = m_s[0];
    }
  }
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

template <typename T, int PER, int CPT, int CHUNK>
static int mlstm_scan_launch(const void* proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                             const float* i_bias, const float* f_bias, float cap, float* S, float* n, float* m,
                             const int* q_start, const int* slot_ids, int num_slots, float* out, int B, int H, int D, int Dv,
                             int seg, int max_segments, void* segments, int* first_of, MlstmScratch scr, int* status,
                             cudaStream_t stream) {
  constexpr int COLS = ML_WARPS * CPT;
  if (D > 32 * PER) return Q3_ERR_SIZE;
  const float q_scale = 1.0f / sqrtf((float)D);
  const dim3 block(ML_THREADS);
  const unsigned slices = (Dv + COLS - 1) / COLS;
  if (seg <= 0) {
    launch(mlstm_scan_kernel<T, PER, CPT, CHUNK, ML_PLAIN>, dim3(slices, H, B), block, 0, stream, (const T*)proj, ld, q_col,
           k_col, v_col, i_col, f_col, i_bias, f_bias, cap, q_scale, S, n, m, q_start, slot_ids, num_slots, out, H, D, Dv,
           (const MlstmSegment*)nullptr, (const int*)nullptr, B, scr, status);
    return launch_status();
  }
  if (B > 1024 || max_segments > 65535) return Q3_ERR_SIZE;
  MlstmSegment* list = (MlstmSegment*)segments;
  launch(mlstm_segments_kernel, dim3(1), dim3(256), 0, stream, q_start, B, seg, list, first_of, max_segments);
  launch(mlstm_scan_kernel<T, PER, CPT, CHUNK, ML_LOCAL>, dim3(slices, H, max_segments), block, 0, stream, (const T*)proj, ld,
         q_col, k_col, v_col, i_col, f_col, i_bias, f_bias, cap, q_scale, S, n, m, q_start, slot_ids, num_slots, out, H, D, Dv,
         (const MlstmSegment*)list, (const int*)first_of, B, scr, status);
  launch(mlstm_carry_kernel, dim3((D * Dv + 255) / 256, H, B), dim3(256), 0, stream, (const int*)first_of, slot_ids, num_slots,
         (const float*)S, (const float*)n, (const float*)m, scr, H, D, Dv);
  launch(mlstm_scan_kernel<T, PER, CPT, CHUNK, ML_FINAL>, dim3(slices, H, max_segments), block, 0, stream, (const T*)proj, ld,
         q_col, k_col, v_col, i_col, f_col, i_bias, f_bias, cap, q_scale, S, n, m, q_start, slot_ids, num_slots, out, H, D, Dv,
         (const MlstmSegment*)list, (const int*)first_of, B, scr, status);
  return launch_status();
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

// The largest key size the scan takes.
extern "C" int q3_mlstm_max_dim() { return 512; }

// proj: [T, ld] in `dtype` with q and k (H * D each), v (H * Dv) and the gates' pre-activations (H each) at the given
// columns; i_bias, f_bias: float32 [H]; S [slots, H, Dv, D] (column by column), n [slots, H, D], m [slots, H]: float32
// state; out: float32 [T, H * Dv].  q is multiplied by D^-1/2.
// seg > 0: the segmented form with segments of `seg` tokens, for which the caller gives scratch for max_segments >=
// T / seg + B segments: `segments` (16 bytes each), first_of (int32 [B + 1]), scratch_S [max_segments, H, Dv, D],
// scratch_n [max_segments, H, D] and scratch_m [3, max_segments, H].
extern "C" int q3_mlstm_scan(const void* proj, int ld, int q_col, int k_col, int v_col, int i_col, int f_col,
                             const float* i_bias, const float* f_bias, float cap, float* S, float* n, float* m,
                             const int* q_start, const int* slot_ids, int num_slots, float* out, int dtype, int B, int H,
                             int D, int Dv, int seg, int max_segments, void* segments, int* first_of, float* scratch_S,
                             float* scratch_n, float* scratch_m, int* status, cudaStream_t stream) {
  if (B <= 0) return 0;
  if (H <= 0 || H > 65535 || B > 65535 || D <= 0 || D > 512 || Dv <= 0 || cap <= 0.f || num_slots <= 0) return Q3_ERR_SIZE;
  q3::MlstmScratch scr{scratch_S, scratch_n, scratch_m, nullptr, nullptr};
  if (seg > 0) {
    if (!segments || !first_of || !scratch_S || !scratch_n || !scratch_m || max_segments <= 0) return Q3_ERR_SCRATCH;
    scr.F = scratch_m + (size_t)max_segments * H;
    scr.m_in = scratch_m + (size_t)2 * max_segments * H;
  }
  // rows of a column per lane by the key size; as many columns per warp as leave 32 values of S per lane; a chunk is
  // as many tokens as the threads can fetch ahead (chunk * D <= 1024)
#define Q3_ML(PER, CPT, CHUNK)                                                                                         \
  Q3_BY_DTYPE(dtype, return (q3::mlstm_scan_launch<E, PER, CPT, CHUNK>(proj, ld, q_col, k_col, v_col, i_col, f_col, i_bias, \
                                                                       f_bias, cap, S, n, m, q_start, slot_ids, num_slots, \
                                                                       out, B, H, D, Dv, seg, max_segments, segments,       \
                                                                       first_of, scr, status, stream)))
  if (D <= 32) { Q3_ML(1, 8, 8) }
  if (D <= 64) { Q3_ML(2, 8, 8) }
  if (D <= 128) { Q3_ML(4, 8, 8) }
  if (D <= 256) { Q3_ML(8, 4, 4) }
  Q3_ML(16, 2, 2)
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
