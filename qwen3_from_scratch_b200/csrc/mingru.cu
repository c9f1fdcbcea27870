// minGRU: a gated recurrence whose gates read only the current token.  With the projections z', u', g' of the mixer's
// input (columns of one product) and biases bz, bu:
//
//   z = sigmoid(z' + bz);   u = u' + bu;   candidate = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//   S_t = (1 - z) S_(t-1) + z candidate          element by element, S in float32, zero for a new request
//   out_t = S_t silu(g') out_scale
//
// mingru_scan: one thread per (request, channel) walks the request's tokens of the step in order; the state slot is
// read once and written once.  Everything but the projections is float32.
#include "common.cuh"

namespace q3 {

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

}  // namespace q3

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
