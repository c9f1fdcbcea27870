// A feed-forward of routed experts: every token goes through `top` of E small feed-forwards W_down act(W_up h),
// chosen by a router, and the results are added with the router's weights.
//
//   moe_route      logits z = W_r h in float32, scores s = sigmoid(z); the `top` experts with the largest s + bias[e]
//                  are chosen (ties: the lower index), their weights are s * scale (the bias takes no part in the
//                  weights, nothing is renormalised).  One block per token.
//   moe_pair_up    for every (token, chosen expert) pair: act(W_up[e] h), a warp per output value; the pair's expert
//                  weight is streamed once per pair.  For a few tokens (decoding) and the float32 run.
//   moe_pair_down  out[t] = base[t] + sum_k weight[t, k] W_down[e_k] a[t, k]: a warp per output value, the chosen
//                  experts in the order the router listed them.
//
// Gated experts (`gate_block` > 0): W_down (act(W_gate h) * (W_up h)); the stack `up` then holds 2 F rows per
// expert, gate and up rows alternating in blocks of `gate_block` rows (gate_block = F: all gate rows, then all up
// rows).  `in_wts` (or null): the router's weight multiplies what the expert reads (both of its first products)
// instead of what it returns; the caller then passes ones as `wts` to the second kernel.
//
// Sums over a row are taken lane by lane in ascending order and then across the warp, so a token's result does not
// depend on the batch.  The expert weights are stacked: up [E, F, W], down [E, W, F].
#include "common.cuh"

namespace q3 {

constexpr int MOE_MAX_TOP = 32;

__device__ __forceinline__ void load4(const float* p, float (&x)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  x[0] = v.x, x[1] = v.y, x[2] = v.z, x[3] = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&x)[4]) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  x[0] = a.x, x[1] = a.y, x[2] = b.x, x[3] = b.y;
}

template <typename T>
__global__ void moe_route_kernel(const T* __restrict__ h, const float* __restrict__ wr, const float* __restrict__ bias,
                                 int* __restrict__ ids, float* __restrict__ wts, int W, int E, int top, float scale) {
  extern __shared__ float score[];  // [E] scores, then [E] choice scores
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  const T* row = h + (size_t)t * W;
  // four values per lane and turn where the rows allow it, so that a warp has its loads in flight together
  const bool by4 = (W & 3) == 0 && ((uintptr_t)row & (4 * sizeof(T) - 1)) == 0 && ((uintptr_t)wr & 15) == 0;
  for (int e = warp; e < E; e += nwarps) {
    const float* w = wr + (size_t)e * W;
    float dot = 0.f;
    if (by4) {
#pragma unroll 8
      for (int i = 4 * lane; i < W; i += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(w + i);
        float x[4];
        load4(row + i, x);
        dot = fmaf(x[0], wv.x, dot);
        dot = fmaf(x[1], wv.y, dot);
        dot = fmaf(x[2], wv.z, dot);
        dot = fmaf(x[3], wv.w, dot);
      }
    } else {
      for (int i = lane; i < W; i += 32) dot = fmaf(to_float(row[i]), w[i], dot);
    }
    dot = warp_sum(dot);
    if (lane == 0) {
      const float s = 1.0f / (1.0f + expf(-dot));
      score[e] = s;
      score[E + e] = s + (bias ? bias[e] : 0.f);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int k = 0; k < top; ++k) {
      int best = -1;
      float bv = -INFINITY;
      for (int e = 0; e < E; ++e) {
        const float v = score[E + e];
        if (v > bv || (best < 0 && !(v < bv))) {  // the second clause takes a NaN rather than nothing
          bv = v;
          best = e;
        }
      }
      ids[(size_t)t * top + k] = best;
      wts[(size_t)t * top + k] = score[best] * scale;
      score[E + best] = -INFINITY;
    }
  }
}

// grid (pairs, ceil(F / warps)).  a[pair, f] = act(sum_i up[e, f, i] h[t, i]), t = pair / top.
template <typename T>
__global__ void moe_pair_up_kernel(const T* __restrict__ h, const T* __restrict__ up, const int* __restrict__ ids,
                                   T* __restrict__ a, int W, int F, int E, int top, int act, int gate_block,
                                   const float* __restrict__ in_wts) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int f = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int pair = blockIdx.x;
  if (f >= F) return;
  const int e = ids[pair];
  if (e < 0 || e >= E) {
    if (lane == 0) a[(size_t)pair * F + f] = from_float<T>(0.f);
    return;
  }
  const T* row = h + (size_t)(pair / top) * W;
  const float in_scale = in_wts ? in_wts[pair] : 1.f;
  if (gate_block > 0) {
    const size_t gate_row = (size_t)(f / gate_block) * 2 * gate_block + f % gate_block;
    const T* wg = up + ((size_t)e * 2 * F + gate_row) * W;
    const T* wu = wg + (size_t)gate_block * W;
    float dg = 0.f, du = 0.f;
    for (int i = lane; i < W; i += 32) {
      const float x = to_float(row[i]);
      dg = fmaf(x, to_float(wg[i]), dg);
      du = fmaf(x, to_float(wu[i]), du);
    }
    dg = warp_sum(dg) * in_scale;
    du = warp_sum(du) * in_scale;
    if (lane == 0) a[(size_t)pair * F + f] = from_float<T>(activate(dg, act) * du);
    return;
  }
  const T* w = up + ((size_t)e * F + f) * W;
  float dot = 0.f;
  for (int i = lane; i < W; i += 32) dot = fmaf(to_float(row[i]), to_float(w[i]), dot);
  dot = warp_sum(dot) * in_scale;
  if (lane == 0) a[(size_t)pair * F + f] = from_float<T>(activate(dot, act));
}

// grid (T, ceil(W / warps)).  out[t, c] = base[t, c] + sum_k wts[t, k] sum_f down[e_k, c, f] a[t * top + k, f].
template <typename T>
__global__ void moe_pair_down_kernel(const T* __restrict__ a, const T* __restrict__ down, const int* __restrict__ ids,
                                     const float* __restrict__ wts, const T* __restrict__ base, T* __restrict__ out, int W,
                                     int F, int E, int top) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int c = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int t = blockIdx.x;
  if (c >= W) return;
  float acc = base ? to_float(base[(size_t)t * W + c]) : 0.f;
  for (int k = 0; k < top; ++k) {
    const int e = ids[(size_t)t * top + k];
    if (e < 0 || e >= E) continue;
    const T* row = a + ((size_t)t * top + k) * F;
    const T* w = down + ((size_t)e * W + c) * F;
    float dot = 0.f;
    for (int i = lane; i < F; i += 32) dot = fmaf(to_float(row[i]), to_float(w[i]), dot);
    acc = fmaf(wts[(size_t)t * top + k], warp_sum(dot), acc);
  }
  if (lane == 0) out[(size_t)t * W + c] = from_float<T>(acc);
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E_ = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E_ = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

// h: [T, W] in `dtype`; wr: float32 [E, W]; bias: float32 [E] or null; ids: int32 [T, top]; wts: float32 [T, top].
extern "C" int q3_moe_route(const void* h, const float* wr, const float* bias, int* ids, float* wts, int dtype, int T, int W,
                            int E, int top, float scale, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (W <= 0 || E <= 0 || top <= 0 || top > E || top > q3::MOE_MAX_TOP || E > 4096) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::moe_route_kernel<E_>, dim3(T), dim3(E >= 16 ? 512 : (E >= 8 ? 256 : 128)), (size_t)2 * E * sizeof(float),
                                stream,
                                (const E_*)h, wr, bias, ids, wts, W, E, top, scale))
  return q3::launch_status();
}

// a: [T * top, F] = act(up[ids] h); out: [T, W] = base + sum_k wts down[ids] a.  act: a Q3_ACT_* code.
// gate_block > 0: gated experts (see the head of the file); in_wts: float32 [T * top] or null.
extern "C" int q3_moe_pairs(const void* h, const void* up, const void* down, const int* ids, const float* wts,
                            const void* base, void* a, void* out, int dtype, int T, int W, int F, int E, int top, int act,
                            int gate_block, const float* in_wts, cudaStream_t stream) {
  if (gate_block < 0 || (gate_block > 0 && F % gate_block)) return Q3_ERR_SIZE;
  if (T <= 0) return 0;
  if (W <= 0 || F <= 0 || E <= 0 || top <= 0 || (long long)T * top > 0x7fffffffll || F > 4 * 65535 || W > 4 * 65535 || act < 0 || act > Q3_ACT_RELU_SQ)
    return Q3_ERR_SIZE;
  const int warps = 4;
  Q3_BY_DTYPE(dtype, q3::launch(q3::moe_pair_up_kernel<E_>, dim3(T * top, (F + warps - 1) / warps), dim3(warps * 32), 0,
                                stream, (const E_*)h, (const E_*)up, ids, (E_*)a, W, F, E, top, act, gate_block, in_wts))
  int code = q3::launch_status();
  if (code) return code;
  Q3_BY_DTYPE(dtype, q3::launch(q3::moe_pair_down_kernel<E_>, dim3(T, (W + warps - 1) / warps), dim3(warps * 32), 0, stream,
                                (const E_*)a, (const E_*)down, ids, wts, (const E_*)base, (E_*)out, W, F, E, top))
  return q3::launch_status();
}
