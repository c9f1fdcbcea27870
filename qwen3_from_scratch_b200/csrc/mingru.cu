// minGRU: a gated recurrence whose gates read only the current token.  With the projections z', u', g' of the mixer's
// input (columns of one product) and biases bz, bu:
//
//   z = sigmoid(z' + bz);   u = u' + bu;   candidate = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//   S_t = (1 - z) S_(t-1) + z candidate          element by element, S in float32, zero for a new request
//   out_t = S_t silu(g') out_scale
//
// mingru_scan: one thread per (request, channel) walks the request's tokens of the step in order; the state slot is
// read once and written once.  Everything but the projections is float32.
//
// mingru_scan_chunked (bfloat16 run, long portions): the recurrence is linear in the state, S_t = a_t S_(t-1) + b_t
// with a = 1 - z and b = z candidate, so a portion is cut into chunks of MG_CHUNK tokens that run side by side: a
// first pass leaves every chunk's product of a and the state it reaches from zero, a carry kernel walks the chunks
// of each request and leaves every chunk's incoming state (and the request's new state), and a third pass walks
// each chunk again from there and writes the output.  Chunk j of request b is filed at scratch record
// q_start[b] / MG_CHUNK + b + j, which never collides.  The sums differ from the single walk's by float32 rounding;
// the float32 run keeps the single walk.
#include "common.cuh"

namespace q3 {

constexpr int MG_CHUNK = 32;

template <typename T>
__global__ void mingru_scan_kernel(const T* __restrict__ proj, int ld, int z_col, int u_col, int g_col,
                                   const float* __restrict__ bz, const float* __restrict__ bu, float* __restrict__ state,
                                   const int* __restrict__ q_start, const int* __restrict__ slot_ids, T* __restrict__ out,
                                   int ldo, int B, int C, int slots, float out_scale, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C || b >= B) return;
  const int slot = slot_ids[b];
  const int s0 = q_start[b], s1 = q_start[b + 1];
  if (slot < 0 || slot >= slots) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    for (int t = s0; t < s1; ++t) out[(size_t)t * ldo + c] = from_float<T>(0.f);
    return;
  }
  float S = state[(size_t)slot * C + c];
  const float zb = bz[c], ub = bu[c];
  for (int t = s0; t < s1; ++t) {
    const T* row = proj + (size_t)t * ld;
    const float z = sigmoid_f(to_float(row[z_col + c]) + zb);
    const float u = to_float(row[u_col + c]) + ub;
    const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
    S = fmaf(z, cand - S, S);  // (1 - z) S + z cand
    out[(size_t)t * ldo + c] = from_float<T>(S * silu_f(to_float(row[g_col + c])) * out_scale);
  }
  state[(size_t)slot * C + c] = S;
}

// The bfloat16 run's sigmoid: the hardware's exponential and reciprocal (float32 arithmetic, relative error near 2^-21).
__device__ __forceinline__ float mg_sigmoid(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

// grid (requests, chunks, channel groups).  PASS 1: scratch [record][0][C] = product of (1 - z), [record][1][C] = the
// state reached from zero.  PASS 3: walks from scratch [record][0][C] (the incoming state) and writes the output.
template <typename T, int PASS>
__global__ void mingru_chunk_kernel(const T* __restrict__ proj, int ld, int z_col, int u_col, int g_col,
                                    const float* __restrict__ bz, const float* __restrict__ bu, float* __restrict__ scratch,
                                    const int* __restrict__ q_start, T* __restrict__ out, int ldo, int C, float out_scale) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, j = blockIdx.y;
  const int c = blockIdx.z * blockDim.x + threadIdx.x;
  const int t0 = q_start[b] + j * MG_CHUNK, end = q_start[b + 1];
  if (c >= C || t0 >= end) return;
  const int t1 = min(end, t0 + MG_CHUNK);
  float* sc = scratch + ((size_t)(q_start[b] / MG_CHUNK + b + j) * 2) * C + c;
  const float zb = bz[c], ub = bu[c];
  float S = PASS == 3 ? sc[0] : 0.f, P = 1.f;
#pragma unroll 8
  for (int t = t0; t < t1; ++t) {
    const T* row = proj + (size_t)t * ld;
    const float z = mg_sigmoid(to_float(row[z_col + c]) + zb);
    const float u = to_float(row[u_col + c]) + ub;
    const float cand = u >= 0.f ? u + 0.5f : mg_sigmoid(u);
    S = fmaf(z, cand - S, S);
    if (PASS == 1) P *= 1.0f - z;
    if (PASS == 3) {
      const float g = to_float(row[g_col + c]);
      out[(size_t)t * ldo + c] = from_float<T>(S * g * mg_sigmoid(g) * out_scale);
    }
  }
  if (PASS == 1) {
    sc[0] = P;
    sc[C] = S;
  }
}

// grid (requests, channel groups): scratch [record][0] becomes the chunk's incoming state; the request's slot receives
// the state after its last chunk.
__global__ void mingru_carry_kernel(float* __restrict__ scratch, float* __restrict__ state, const int* __restrict__ q_start,
                                    const int* __restrict__ slot_ids, int C, int slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int slot = slot_ids[b];
  const bool live = slot >= 0 && slot < slots;
  if (!live && threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
  const int n = q_start[b + 1] - q_start[b];
  const int chunks = (n + MG_CHUNK - 1) / MG_CHUNK;
  float* sc = scratch + ((size_t)(q_start[b] / MG_CHUNK + b) * 2) * C + c;
  float S = live ? state[(size_t)slot * C + c] : 0.f;
  for (int j0 = 0; j0 < chunks; j0 += 8) {  // eight records are asked for together, then walked
    float P[8], V[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const bool in = j0 + k < chunks;
      P[k] = in ? sc[(size_t)(j0 + k) * 2 * C] : 1.f;
      V[k] = in ? sc[(size_t)(j0 + k) * 2 * C + C] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (j0 + k < chunks) sc[(size_t)(j0 + k) * 2 * C] = S;
      S = fmaf(P[k], S, V[k]);
    }
  }
  if (live) state[(size_t)slot * C + c] = S;
}

}  // namespace q3

// Tokens per chunk of mingru_scan_chunked; its scratch holds (tokens / chunk + requests + 1) records of 2 C floats.
extern "C" int q3_mingru_chunk() { return q3::MG_CHUNK; }

// The same recurrence as q3_mingru_scan over chunks of the portions (three launches), bfloat16 only.
extern "C" int q3_mingru_scan_chunked(const void* proj, int ld, int z_col, int u_col, int g_col, const float* bz,
                                      const float* bu, float* state, float* scratch, const int* q_start,
                                      const int* slot_ids, void* out, int ldo, int dtype, int T, int B, int max_q_len, int C,
                                      int slots, float out_scale, int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0 || max_q_len <= 0) return 0;
  if (dtype != Q3_BF16) return Q3_ERR_DTYPE;
  const int threads = 64;
  const int chunks = (max_q_len + q3::MG_CHUNK - 1) / q3::MG_CHUNK;
  const dim3 grid(B, chunks, (C + threads - 1) / threads), cgrid(B, (C + threads - 1) / threads);
  if (C <= 0 || chunks > 65535 || grid.z > 65535) return Q3_ERR_SIZE;
  using E = __nv_bfloat16;
  q3::launch(q3::mingru_chunk_kernel<E, 1>, grid, dim3(threads), 0, stream, (const E*)proj, ld, z_col, u_col, g_col, bz, bu,
             scratch, q_start, (E*)out, ldo, C, out_scale);
  q3::launch(q3::mingru_carry_kernel, cgrid, dim3(threads), 0, stream, scratch, state, q_start, slot_ids, C, slots, status);
  q3::launch(q3::mingru_chunk_kernel<E, 3>, grid, dim3(threads), 0, stream, (const E*)proj, ld, z_col, u_col, g_col, bz, bu,
             scratch, q_start, (E*)out, ldo, C, out_scale);
  return q3::launch_status();
}

// proj: [T, ld] in `dtype` with the three projections of C channels at columns z_col, u_col, g_col; state: float32
// [slots, C]; out: rows of `ldo` values in `dtype` (the channels at the pointer given).
extern "C" int q3_mingru_scan(const void* proj, int ld, int z_col, int u_col, int g_col, const float* bz, const float* bu,
                              float* state, const int* q_start, const int* slot_ids, void* out, int ldo, int dtype, int T,
                              int B, int C, int slots, float out_scale, int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return 0;
  if (C <= 0 || B > 65535) return Q3_ERR_SIZE;
  const int threads = 64;
  const dim3 grid((C + threads - 1) / threads, B);
  if (dtype == Q3_F32)
    q3::launch(q3::mingru_scan_kernel<float>, grid, dim3(threads), 0, stream, (const float*)proj, ld, z_col, u_col, g_col,
               bz, bu, state, q_start, slot_ids, (float*)out, ldo, B, C, slots, out_scale, status);
  else if (dtype == Q3_BF16)
    q3::launch(q3::mingru_scan_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)proj, ld, z_col,
               u_col, g_col, bz, bu, state, q_start, slot_ids, (__nv_bfloat16*)out, ldo, B, C, slots, out_scale, status);
  else
    return Q3_ERR_DTYPE;
  return q3::launch_status();
}
