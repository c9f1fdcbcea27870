// Layer norm with weight and bias around the float32 residual stream, and the short causal convolution that a
// block may put in front of a sub-layer.
//
//   add_layernorm        stream += delta (in place, float32), out = (x - mean) / sqrt(var + eps) * w + b, where var is
//                        the mean of the squared deviations; statistics in float32 in two passes over the row, which
//                        the block keeps in shared memory.  With `rows` the kernel norms chosen rows and leaves the
//                        stream as it is (the model's last norm).  The result is float32 or the compute dtype.
//   input_conv           out[t, c] = h[t, c] + sum_j w[c, j] h[t - (K - 1) + j, c] over the tokens of one request; what
//                        lies before a portion comes from the request's slot of `state` (float32 [slots, K - 1, C],
//                        zero for a new request), which a second launch renews after every reader is done.
//
//   add_layernorm_conv1  both of the above in one launch for a step in which every request brings one token: the
//                        block that norms a token's row applies the convolution from the request's state and
//                        renews the state (each thread reads and writes its own channels of it); same sums, same
//                        order, same bits as the two kernels.
//
//   stream_concat        out[t] = [stream[t] + delta[t] | other[t]] in the compute dtype: the operand of a projection
//                        that reads the stream beside a second float32 tensor of the same shape.
//
// Every sum has an order that depends on the row alone, so a row's result does not depend on what else is in the
// launch.
#include "common.cuh"

namespace q3 {

template <typename TD, typename TO>
__global__ void add_layernorm_kernel(float* __restrict__ stream, const TD* __restrict__ delta, const float* __restrict__ w,
                                     const float* __restrict__ b, TO* __restrict__ out, const int* __restrict__ rows,
                                     int W, float eps) {
  extern __shared__ float row_x[];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t r = rows ? (size_t)rows[blockIdx.x] : (size_t)blockIdx.x;
  float* x = stream + r * W;
  const TD* d = delta ? delta + r * W : nullptr;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = x[i];
    if (d) v += to_float(d[i]);
    if (d && !rows) x[i] = v;
    row_x[i] = v;
    s += v;
  }
  const float mean = block_sum(s, red) / (float)W;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float c = row_x[i] - mean;
    q = fmaf(c, c, q);
  }
  const float inv = 1.0f / sqrtf(block_sum(q, red) / (float)W + eps);
  TO* o = out + (size_t)blockIdx.x * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) o[i] = from_float<TO>((row_x[i] - mean) * inv * w[i] + b[i]);
}

constexpr int CONV_MAX_TAPS = 16;

template <typename TO>
__global__ void input_conv_kernel(const float* __restrict__ h, const float* __restrict__ w, const float* __restrict__ state,
                                  const int* __restrict__ q_start, const int* __restrict__ tok_seq,
                                  const int* __restrict__ slot_ids, TO* __restrict__ out, int T, int C, int K, int slots,
                                  int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t = blockIdx.y;
  if (c >= C) return;
  const int b = tok_seq[t];
  const int s0 = q_start[b], slot = slot_ids[b];
  if (slot < 0 || slot >= slots) {
    if (K > 1) {
      if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
      out[(size_t)t * C + c] = from_float<TO>(0.f);
      return;
    }
  }
  float acc = h[(size_t)t * C + c];
  for (int j = 0; j < K; ++j) {
    const int src = t - (K - 1) + j;
    const float v = src >= s0 ? h[(size_t)src * C + c]
                              : state[((size_t)slot * (K - 1) + (K - 1 + src - s0)) * C + c];
    acc = fmaf(w[(size_t)c * K + j], v, acc);
  }
  out[(size_t)t * C + c] = from_float<TO>(acc);
}

// The last K - 1 inputs of every request of the step become its new tail: rows of this portion, and, where the
// portion is shorter than the tail, the newest rows of the old tail.  One thread owns a (request, channel) pair and
// reads all it needs before it writes.
__global__ void input_conv_tail_kernel(const float* __restrict__ h, float* __restrict__ state, const int* __restrict__ q_start,
                                       const int* __restrict__ slot_ids, int B, int C, int K, int slots) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C || b >= B) return;
  const int slot = slot_ids[b];
  if (slot < 0 || slot >= slots) return;
  const int s0 = q_start[b], s1 = q_start[b + 1];
  float keep[CONV_MAX_TAPS];
  float* tail = state + (size_t)slot * (K - 1) * C + c;
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i) {
    if (i < K - 1) {
      const int src = s1 - (K - 1) + i;
      keep[i] = src >= s0 ? h[(size_t)src * C + c] : tail[(size_t)(K - 1 + src - s0) * C];
    }
  }
#pragma unroll
  for (int i = 0; i < CONV_MAX_TAPS; ++i)
    if (i < K - 1) tail[(size_t)i * C] = keep[i];
}

template <typename T>
__global__ void stream_concat_kernel(const float* __restrict__ stream, const T* __restrict__ delta,
                                     const float* __restrict__ other, T* __restrict__ out, size_t total, int W) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / (size_t)W;
  const int c = (int)(i - t * W);
  float v = stream[i];
  if (delta) v += to_float(delta[i]);
  out[t * 2 * W + c] = from_float<T>(v);
  out[t * 2 * W + W + c] = from_float<T>(other[i]);
}

template <typename TD, typename TO>
static int add_layernorm_launch(float* stream, const void* delta, const float* w, const float* b, void* out,
                                const int* rows, int n, int W, float eps, cudaStream_t stream_) {
  if (n <= 0) return 0;
  if (W <= 0 || (size_t)W * sizeof(float) > 200 * 1024) return Q3_ERR_SIZE;
  const int threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
  const size_t smem = (size_t)W * sizeof(float);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(add_layernorm_kernel<TD, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch(add_layernorm_kernel<TD, TO>, dim3(n), dim3(threads), smem, stream_, stream, (const TD*)delta, w, b, (TO*)out,
         rows, W, eps);
  if (!rows) note_stream_written();
  return launch_status();
}

}  // namespace q3

namespace q3 {

template <typename TD, typename TO>
__global__ void add_layernorm_conv1_kernel(float* __restrict__ stream, const TD* __restrict__ delta,
                                           const float* __restrict__ w, const float* __restrict__ b,
                                           const float* __restrict__ cw, float* __restrict__ state,
                                           const int* __restrict__ tok_seq, const int* __restrict__ slot_ids,
                                           TO* __restrict__ out, int W, int K, int slots, float eps, int* status) {
  extern __shared__ float row_x[];
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const size_t r = blockIdx.x;
  float* x = stream + r * W;
  const TD* d = delta ? delta + r * W : nullptr;
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = x[i];
    if (d) {
      v += to_float(d[i]);
      x[i] = v;
    }
    row_x[i] = v;
    s += v;
  }
  const float mean = block_sum(s, red) / (float)W;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float c = row_x[i] - mean;
    q = fmaf(c, c, q);
  }
  const float inv = 1.0f / sqrtf(block_sum(q, red) / (float)W + eps);
  const int slot = slot_ids[tok_seq[r]];
  const bool live = K == 1 || (slot >= 0 && slot < slots);
  if (!live && threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
  TO* o = out + r * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    if (!live) {
      o[i] = from_float<TO>(0.f);
      continue;
    }
    const float h = (row_x[i] - mean) * inv * w[i] + b[i];
    float* tail = state + (size_t)slot * (K - 1) * W + i;
    float acc = h;
    for (int j = 0; j < K - 1; ++j) {
      const float v = tail[(size_t)j * W];
      acc = fmaf(cw[(size_t)i * K + j], v, acc);
      if (j > 0) tail[(size_t)(j - 1) * W] = v;
    }
    acc = fmaf(cw[(size_t)i * K + K - 1], h, acc);
    if (K > 1) tail[(size_t)(K - 2) * W] = h;
    o[i] = from_float<TO>(acc);
  }
}

}  // namespace q3

// stream: float32 [T, W] (+= delta in place); out [T, W] in `dtype` = h + conv(h) for h = layer norm of the row, every
// request of the step bringing exactly one token; cw: float32 [W, K]; state: float32 [slots, K - 1, W], renewed.
extern "C" int q3_add_layernorm_conv1(float* stream, const void* delta, const float* w, const float* b, const float* cw,
                                      float* state, const int* tok_seq, const int* slot_ids, void* out, int dtype, int T,
                                      int W, int K, int slots, float eps, int* status, cudaStream_t stream_) {
  if (T <= 0) return 0;
  if (W <= 0 || K <= 0 || K > q3::CONV_MAX_TAPS || (size_t)W * sizeof(float) > 200 * 1024) return Q3_ERR_SIZE;
  const int threads = W >= 2048 ? 512 : (W >= 512 ? 256 : 128);
  const size_t smem = (size_t)W * sizeof(float);
  if (dtype == Q3_F32) {
    auto kern = q3::add_layernorm_conv1_kernel<float, float>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    q3::launch(kern, dim3(T), dim3(threads), smem, stream_, stream, (const float*)delta, w, b, cw, state, tok_seq, slot_ids,
               (float*)out, W, K, slots, eps, status);
  } else if (dtype == Q3_BF16) {
    auto kern = q3::add_layernorm_conv1_kernel<__nv_bfloat16, __nv_bfloat16>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    q3::launch(kern, dim3(T), dim3(threads), smem, stream_, stream, (const __nv_bfloat16*)delta, w, b, cw, state, tok_seq,
               slot_ids, (__nv_bfloat16*)out, W, K, slots, eps, status);
  } else {
    return Q3_ERR_DTYPE;
  }
  q3::note_stream_written();
  return q3::launch_status();
}

// stream: float32 [T, W], += delta (compute dtype `dtype`, may be null) in place unless `rows` is given; out [n, W] in
// float32 (`out_f32`) or in `dtype`; n = number of rows normed (T, or the length of `rows`).
extern "C" int q3_add_layernorm(float* stream, const void* delta, const float* w, const float* b, void* out, int out_f32,
                                int dtype, const int* rows, int n, int W, float eps, cudaStream_t s) {
  if (dtype == Q3_F32) return q3::add_layernorm_launch<float, float>(stream, delta, w, b, out, rows, n, W, eps, s);
  if (dtype != Q3_BF16) return Q3_ERR_DTYPE;
  if (out_f32) return q3::add_layernorm_launch<__nv_bfloat16, float>(stream, delta, w, b, out, rows, n, W, eps, s);
  return q3::add_layernorm_launch<__nv_bfloat16, __nv_bfloat16>(stream, delta, w, b, out, rows, n, W, eps, s);
}

// h: float32 [T, C]; w: float32 [C, K]; state: float32 [slots, K - 1, C] (unused for K = 1); out [T, C] in `dtype`.
namespace q3 {

// The same sums for four channels per thread (C a multiple of 4, 16-byte aligned rows): one 16-byte load per tap.
template <typename TO>
__global__ void input_conv_vec4_kernel(const float* __restrict__ h, const float* __restrict__ w,
                                       const float* __restrict__ state, const int* __restrict__ q_start,
                                       const int* __restrict__ tok_seq, const int* __restrict__ slot_ids,
                                       TO* __restrict__ out, int T, int C, int K, int slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
  const int t = blockIdx.y;
  if (c >= C) return;
  const int b = tok_seq[t];
  const int s0 = q_start[b], slot = slot_ids[b];
  TO* o = out + (size_t)t * C + c;
  if (K > 1 && (slot < 0 || slot >= slots)) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = from_float<TO>(0.f);
    return;
  }
  const float4 own = *reinterpret_cast<const float4*>(h + (size_t)t * C + c);
  float acc[4] = {own.x, own.y, own.z, own.w};
  for (int j = 0; j < K; ++j) {
    const int src = t - (K - 1) + j;
    const float4 v = *reinterpret_cast<const float4*>(
        src >= s0 ? h + (size_t)src * C + c : state + ((size_t)slot * (K - 1) + (K - 1 + src - s0)) * C + c);
    acc[0] = fmaf(w[(size_t)(c + 0) * K + j], v.x, acc[0]);
    acc[1] = fmaf(w[(size_t)(c + 1) * K + j], v.y, acc[1]);
    acc[2] = fmaf(w[(size_t)(c + 2) * K + j], v.z, acc[2]);
    acc[3] = fmaf(w[(size_t)(c + 3) * K + j], v.w, acc[3]);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = from_float<TO>(acc[i]);
}

// The same sums again for a run of CONV_RUN tokens and four channels per thread, K known at compile time: the run's
// rows and the K - 1 before it are asked for at once and stay in registers, so that a row is loaded once per run
// instead of once per tap; a token whose portion starts inside the window takes the older rows from the state.
constexpr int CONV_RUN = 8;

template <typename TO, int K>
__global__ void input_conv_run_kernel(const float* __restrict__ h, const float* __restrict__ w,
                                      const float* __restrict__ state, const int* __restrict__ q_start,
                                      const int* __restrict__ tok_seq, const int* __restrict__ slot_ids,
                                      TO* __restrict__ out, int T, int C, int slots, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  const int c = 4 * (blockIdx.x * blockDim.x + threadIdx.x);
  const int t0 = blockIdx.y * CONV_RUN;
  if (c >= C) return;
  float4 win[CONV_RUN + K - 1];
#pragma unroll
  for (int i = 0; i < CONV_RUN + K - 1; ++i) {
    const int src = t0 - (K - 1) + i;
    win[i] = (src >= 0 && src < T) ? *reinterpret_cast<const float4*>(h + (size_t)src * C + c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  float wk[4][K];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < K; ++j) wk[i][j] = w[(size_t)(c + i) * K + j];
#pragma unroll
  for (int r = 0; r < CONV_RUN; ++r) {
    const int t = t0 + r;
    if (t >= T) break;
    const int b = tok_seq[t];
    const int s0 = q_start[b], slot = slot_ids[b];
    TO* o = out + (size_t)t * C + c;
    const bool live = K == 1 || (slot >= 0 && slot < slots);
    if (!live) {
      if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
#pragma unroll
      for (int i = 0; i < 4; ++i) o[i] = from_float<TO>(0.f);
      continue;
    }
    const float4 own = win[r + K - 1];
    float acc[4] = {own.x, own.y, own.z, own.w};
#pragma unroll
    for (int j = 0; j < K; ++j) {
      const int src = t - (K - 1) + j;
      float4 v = win[r + j];
      if (src < s0) v = *reinterpret_cast<const float4*>(state + ((size_t)slot * (K - 1) + (K - 1 + src - s0)) * C + c);
      acc[0] = fmaf(wk[0][j], v.x, acc[0]);
      acc[1] = fmaf(wk[1][j], v.y, acc[1]);
      acc[2] = fmaf(wk[2][j], v.z, acc[2]);
      acc[3] = fmaf(wk[3][j], v.w, acc[3]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) o[i] = from_float<TO>(acc[i]);
  }
}

template <typename TO>
static bool input_conv_run_launch(const float* h, const float* w, const float* state, const int* q_start, const int* tok_seq,
                                  const int* slot_ids, void* out, int T, int C, int K, int slots, int* status,
                                  cudaStream_t stream) {
  const int threads = 64;
  const dim3 grid((C / 4 + threads - 1) / threads, (T + CONV_RUN - 1) / CONV_RUN);
#define Q3_CONV_RUN_CASE(KK)                                                                                       \
  if (K == KK) {                                                                                                   \
    launch(input_conv_run_kernel<TO, KK>, grid, dim3(threads), 0, stream, h, w, state, q_start, tok_seq, slot_ids, \
           (TO*)out, T, C, slots, status);                                                                         \
    return true;                                                                                                   \
  }
  Q3_CONV_RUN_CASE(2) Q3_CONV_RUN_CASE(3) Q3_CONV_RUN_CASE(4) Q3_CONV_RUN_CASE(5) Q3_CONV_RUN_CASE(6) Q3_CONV_RUN_CASE(7)
  Q3_CONV_RUN_CASE(8)
#undef Q3_CONV_RUN_CASE
  return false;
}

}  // namespace q3

extern "C" int q3_input_conv(const float* h, const float* w, float* state, const int* q_start, const int* tok_seq,
                             const int* slot_ids, void* out, int dtype, int T, int B, int C, int K, int slots,
                             int renew_state, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (C <= 0 || K <= 0 || K > q3::CONV_MAX_TAPS || B <= 0 || T > 65535 || B > 65535) return Q3_ERR_SIZE;
  const int threads = 128;
  const dim3 grid((C + threads - 1) / threads, T);
  const bool vec4 = C % 4 == 0 && (uintptr_t)h % 16 == 0 && (K == 1 || (uintptr_t)state % 16 == 0);
  const dim3 grid4((C / 4 + threads - 1) / threads, T);
  // many tokens: runs of tokens per thread (taps 2 .. 8)
  const bool runs = vec4 && T >= 4 * q3::CONV_RUN && (dtype == Q3_F32 || dtype == Q3_BF16);
  if (runs && dtype == Q3_F32 &&
      q3::input_conv_run_launch<float>(h, w, (const float*)state, q_start, tok_seq, slot_ids, out, T, C, K, slots, status,
                                       stream)) {
  } else if (runs && dtype == Q3_BF16 &&
             q3::input_conv_run_launch<__nv_bfloat16>(h, w, (const float*)state, q_start, tok_seq, slot_ids, out, T, C, K,
                                                      slots, status, stream)) {
  } else if (vec4 && dtype == Q3_F32)
    q3::launch(q3::input_conv_vec4_kernel<float>, grid4, dim3(threads), 0, stream, h, w, (const float*)state, q_start,
               tok_seq, slot_ids, (float*)out, T, C, K, slots, status);
  else if (vec4 && dtype == Q3_BF16)
    q3::launch(q3::input_conv_vec4_kernel<__nv_bfloat16>, grid4, dim3(threads), 0, stream, h, w, (const float*)state,
               q_start, tok_seq, slot_ids, (__nv_bfloat16*)out, T, C, K, slots, status);
  else if (dtype == Q3_F32)
    q3::launch(q3::input_conv_kernel<float>, grid, dim3(threads), 0, stream, h, w, (const float*)state, q_start, tok_seq,
               slot_ids, (float*)out, T, C, K, slots, status);
  else if (dtype == Q3_BF16)
    q3::launch(q3::input_conv_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, h, w, (const float*)state, q_start,
               tok_seq, slot_ids, (__nv_bfloat16*)out, T, C, K, slots, status);
  else
    return Q3_ERR_DTYPE;
  int code = q3::launch_status();
  if (code || K == 1 || !renew_state) return code;
  q3::launch(q3::input_conv_tail_kernel, dim3((C + threads - 1) / threads, B), dim3(threads), 0, stream, h, state, q_start,
             slot_ids, B, C, K, slots);
  return q3::launch_status();
}

// stream, other: float32 [T, W]; delta: [T, W] in `dtype` or null; out: [T, 2 W] in `dtype`.
extern "C" int q3_stream_concat(const float* stream, const void* delta, const float* other, void* out, int dtype, int T,
                                int W, cudaStream_t s) {
  if (T <= 0) return 0;
  if (W <= 0) return Q3_ERR_SIZE;
  const size_t total = (size_t)T * W;
  const int threads = 256;
  const size_t blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffull) return Q3_ERR_SIZE;
  if (dtype == Q3_F32)
    q3::launch(q3::stream_concat_kernel<float>, dim3((unsigned)blocks), dim3(threads), 0, s, stream, (const float*)delta,
               other, (float*)out, total, W);
  else if (dtype == Q3_BF16)
    q3::launch(q3::stream_concat_kernel<__nv_bfloat16>, dim3((unsigned)blocks), dim3(threads), 0, s, stream,
               (const __nv_bfloat16*)delta, other, (__nv_bfloat16*)out, total, W);
  else
    return Q3_ERR_DTYPE;
  return q3::launch_status();
}
