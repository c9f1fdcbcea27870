// Dynamic Tanh in place of a norm (Zhu et al., "Transformers without Normalization"): y = tanh(alpha x) w + b with a
// scalar alpha and a weight and bias per feature; no mean, no variance, nothing reduced over the row.  And what a
// block with such "norms" on both sides of every sub-layer does to the float32 residual stream between two products:
//
//   add_dyt        stream += after(delta) + rows_add + vec_add (each part optional; `after` is the Dynamic Tanh that
//                  follows a sub-layer, applied to its output `delta`), then out = before(stream) (`before`: the one
//                  in front of the next sub-layer, or none: out is the stream in the compute dtype); with `rows` the
//                  same for chosen rows only, the stream left as it is (the model's last norm)
//   side_gate      g = gelu_tanh(p) * e: p a product of the stream, e a slice of a token's row of a second embedding
//   add_unit_rms   stream += y / sqrt(mean(y^2) + eps) * w: a product's rows brought to unit root mean square, a
//                  weight per feature, added into the stream
//   sigmoid_gate   x *= sigmoid(g) element by element (an attention's output gate)
//
// All arithmetic float32; alpha is read from device memory (a tensor of the model, no host copy).
#include "common.cuh"

namespace q3 {

struct DytParams {
  const float* alpha;  // one value; null: the identity
  const float* w;
  const float* b;
};

__device__ __forceinline__ float dyt(float x, float alpha, const float* w, const float* b, int c) {
  return fmaf(tanhf(alpha * x), w[c], b[c]);
}

// grid (ceil(W / (4 * 128)) , rows).  `rows` (or null): the rows to work on, the stream then stays as it is.
template <typename T, typename O>
__global__ void add_dyt_kernel(float* __restrict__ stream, const T* __restrict__ delta, DytParams after,
                               const float* __restrict__ rows_add, const float* __restrict__ vec_add, DytParams before,
                               O* __restrict__ out, const int* __restrict__ rows, int W) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.y;
  const int t = rows ? rows[r] : r;
  const float a_after = after.alpha ? *after.alpha : 0.f, a_before = before.alpha ? *before.alpha : 0.f;
  for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < W; c += gridDim.x * blockDim.x) {
    const size_t i = (size_t)t * W + c;
    float x = stream[i];
    if (delta) {
      const float d = to_float(delta[i]);
      x += after.alpha ? dyt(d, a_after, after.w, after.b, c) : d;
    }
    if (rows_add) x += rows_add[i];
    if (vec_add) x += vec_add[c];
    if (!rows) stream[i] = x;
    if (out) out[(size_t)r * W + c] = from_float<O>(before.alpha ? dyt(x, a_before, before.w, before.b, c) : x);
  }
}

// The same four features at a time: 16-byte accesses of the float32 arrays, 8-byte ones of bfloat16 (W a multiple of
// 4, every pointer aligned; the launcher sees to it).  The arithmetic of a feature is add_dyt_kernel's.
__device__ __forceinline__ void load4f(const float* p, float (&x)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  x[0] = v.x, x[1] = v.y, x[2] = v.z, x[3] = v.w;
}
__device__ __forceinline__ void load4f(const __nv_bfloat16* p, float (&x)[4]) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
  x[0] = a.x, x[1] = a.y, x[2] = b.x, x[3] = b.y;
}
__device__ __forceinline__ void store4f(float* p, const float (&x)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
}
__device__ __forceinline__ void store4f(__nv_bfloat16* p, const float (&x)[4]) {
  uint2 v;
  *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(x[0], x[1]);
  *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(x[2], x[3]);
  *reinterpret_cast<uint2*>(p) = v;
}

template <typename T, typename O>
__global__ void add_dyt4_kernel(float* __restrict__ stream, const T* __restrict__ delta, DytParams after,
                                const float* __restrict__ rows_add, const float* __restrict__ vec_add, DytParams before,
                                O* __restrict__ out, const int* __restrict__ rows, int W) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.y;
  const int t = rows ? rows[r] : r;
  const float a_after = after.alpha ? *after.alpha : 0.f, a_before = before.alpha ? *before.alpha : 0.f;
  for (int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4; c < W; c += gridDim.x * blockDim.x * 4) {
    const size_t i = (size_t)t * W + c;
    float x[4], y[4];
    load4f(stream + i, x);
    if (delta) {
      load4f(delta + i, y);
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] += after.alpha ? dyt(y[k], a_after, after.w, after.b, c + k) : y[k];
    }
    if (rows_add) {
      load4f(rows_add + i, y);
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] += y[k];
    }
    if (vec_add) {
#pragma unroll
      for (int k = 0; k < 4; ++k) x[k] += vec_add[c + k];
    }
    if (!rows) store4f(stream + i, x);
    if (out) {
#pragma unroll
      for (int k = 0; k < 4; ++k) y[k] = before.alpha ? dyt(x[k], a_before, before.w, before.b, c + k) : x[k];
      store4f(out + (size_t)r * W + c, y);
    }
  }
}

// A thread per value.  p: [T, dim] in the compute dtype; side: float32 [T, ld], the layer's slice at column `col`.
template <typename T>
__global__ void side_gate_kernel(const T* __restrict__ p, const float* __restrict__ side, int ld, int col,
                                 T* __restrict__ out, int dim, long long total) {
  pdl_wait();
  pdl_launch_dependents();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / dim;
  const int j = (int)(i - t * dim);
  out[i] = from_float<T>(gelu_tanh_f(to_float(p[i])) * side[t * ld + col + j]);
}

// grid (T), one block per row; the sum of squares in the block's fixed order.
template <typename T>
__global__ void add_unit_rms_kernel(float* __restrict__ stream, const T* __restrict__ y, const float* __restrict__ w,
                                    float eps, int W) {
  __shared__ float red[32];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* row = y + (size_t)t * W;
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    const float v = to_float(row[c]);
    ss = fmaf(v, v, ss);
  }
  const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)W + eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) stream[(size_t)t * W + c] += to_float(row[c]) * inv * w[c];
}

// grid (ceil(n / (256 * PER)), T).  x: rows of ldx values, n of them from column 0; g: rows of ldg values, the gates'
// pre-activations from column g_col.  PER values per thread, as one access where the launcher found everything aligned.
template <typename T, int PER>
__global__ void sigmoid_gate_kernel(T* __restrict__ x, int ldx, const T* __restrict__ g, int ldg, int g_col, int n) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.y;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * PER;
  if (c >= n) return;
  struct alignas(sizeof(T) * PER) Pack { T v[PER]; };
  T* xp = x + (size_t)t * ldx + c;
  const T* gp = g + (size_t)t * ldg + g_col + c;
  Pack xv = *reinterpret_cast<const Pack*>(xp);
  const Pack gv = *reinterpret_cast<const Pack*>(gp);
#pragma unroll
  for (int i = 0; i < PER; ++i) xv.v[i] = from_float<T>(to_float(xv.v[i]) * sigmoid_f(to_float(gv.v[i])));
  *reinterpret_cast<Pack*>(xp) = xv;
}

}  // namespace q3

#define Q3_BY_DTYPE(dtype, CALL)                 \
  if ((dtype) == Q3_F32) { using E = float; CALL; }  \
  else if ((dtype) == Q3_BF16) { using E = __nv_bfloat16; CALL; } \
  else return Q3_ERR_DTYPE;

// stream: float32 [T, W]; delta: [T, W] in `dtype` or null; after_* / before_*: alpha (one float32 on the device),
// weight and bias (float32 [W]) of the Dynamic Tanh after the sub-layer / before the next, alpha null for none;
// rows_add: float32 [T, W] or null; vec_add: float32 [W] or null; out: [R, W] in `dtype` (float32 with out_f32) or
// null; rows: int32 [R] or null (then R = T and the stream is updated).
extern "C" int q3_add_dyt(float* stream, const void* delta, const float* after_alpha, const float* after_w,
                          const float* after_b, const float* rows_add, const float* vec_add, const float* before_alpha,
                          const float* before_w, const float* before_b, void* out, int out_f32, const int* rows, int R,
                          int dtype, int T, int W, cudaStream_t cuda_stream) {
  const int n = rows ? R : T;
  if (n <= 0) return 0;
  if (W <= 0) return Q3_ERR_SIZE;
  const q3::DytParams after{after_alpha, after_w, after_b}, before{before_alpha, before_w, before_b};
  const dim3 grid((unsigned)((W + 1023) / 1024 > 0 ? (W + 1023) / 1024 : 1), (unsigned)n), block(256);
  if (n > 65535) return Q3_ERR_SIZE;
  const bool by4 = W % 4 == 0 && (uintptr_t)stream % 16 == 0 && (uintptr_t)delta % 16 == 0 && (uintptr_t)rows_add % 16 == 0 &&
                   (uintptr_t)out % 16 == 0;
  if (by4) {  // the same arithmetic, four features per access
    if (out_f32) {
      Q3_BY_DTYPE(dtype, q3::launch(q3::add_dyt4_kernel<E, float>, grid, block, 0, cuda_stream, stream, (const E*)delta,
                                    after, rows_add, vec_add, before, (float*)out, rows, W))
    } else {
      Q3_BY_DTYPE(dtype, q3::launch(q3::add_dyt4_kernel<E, E>, grid, block, 0, cuda_stream, stream, (const E*)delta, after,
                                    rows_add, vec_add, before, (E*)out, rows, W))
    }
    if (!rows) q3::note_stream_written();
    return q3::launch_status();
  }
  if (out_f32) {
    Q3_BY_DTYPE(dtype, q3::launch(q3::add_dyt_kernel<E, float>, grid, block, 0, cuda_stream, stream, (const E*)delta, after,
                                  rows_add, vec_add, before, (float*)out, rows, W))
  } else {
    Q3_BY_DTYPE(dtype, q3::launch(q3::add_dyt_kernel<E, E>, grid, block, 0, cuda_stream, stream, (const E*)delta, after,
                                  rows_add, vec_add, before, (E*)out, rows, W))
  }
  if (!rows) q3::note_stream_written();
  return q3::launch_status();
}

extern "C" int q3_side_gate(const void* p, const float* side, int ld, int col, void* out, int dtype, int T, int dim,
                            cudaStream_t stream) {
  if (T <= 0) return 0;
  if (dim <= 0 || col < 0 || col + dim > ld) return Q3_ERR_SIZE;
  const long long total = (long long)T * dim;
  if ((total + 255) / 256 > 0x7fffffffll) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::side_gate_kernel<E>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream,
                                (const E*)p, side, ld, col, (E*)out, dim, total))
  return q3::launch_status();
}

extern "C" int q3_add_unit_rms(float* stream, const void* y, const float* w, float eps, int dtype, int T, int W,
                               cudaStream_t cuda_stream) {
  if (T <= 0) return 0;
  if (W <= 0) return Q3_ERR_SIZE;
  Q3_BY_DTYPE(dtype, q3::launch(q3::add_unit_rms_kernel<E>, dim3(T), dim3(W >= 1024 ? 256 : 128), 0, cuda_stream, stream,
                                (const E*)y, w, eps, W))
  q3::note_stream_written();
  return q3::launch_status();
}

extern "C" int q3_sigmoid_gate(void* x, int ldx, const void* g, int ldg, int g_col, int n, int dtype, int T,
                               cudaStream_t stream) {
  if (T <= 0 || n <= 0) return 0;
  if (T > 65535 || ldx < n || g_col < 0 || g_col + n > ldg) return Q3_ERR_SIZE;
  // 16 bytes per access where the columns, the row pitches and the pointers allow it
  const size_t es = dtype == Q3_F32 ? 4 : 2;
  const int per = (int)(16 / es);
  const bool wide = n % per == 0 && ldx % per == 0 && ldg % per == 0 && g_col % per == 0 && (uintptr_t)x % 16 == 0 &&
                    (uintptr_t)g % 16 == 0;
  if (wide) {
    if (dtype == Q3_F32)
      q3::launch(q3::sigmoid_gate_kernel<float, 4>, dim3((n / 4 + 255) / 256, T), dim3(256), 0, stream, (float*)x, ldx,
                 (const float*)g, ldg, g_col, n);
    else if (dtype == Q3_BF16)
      q3::launch(q3::sigmoid_gate_kernel<__nv_bfloat16, 8>, dim3((n / 8 + 255) / 256, T), dim3(256), 0, stream,
                 (__nv_bfloat16*)x, ldx, (const __nv_bfloat16*)g, ldg, g_col, n);
    else
      return Q3_ERR_DTYPE;
    return q3::launch_status();
  }
  Q3_BY_DTYPE(dtype, q3::launch(q3::sigmoid_gate_kernel<E, 1>, dim3((n + 255) / 256, T), dim3(256), 0, stream, (E*)x, ldx,
                                (const E*)g, ldg, g_col, n))
  return q3::launch_status();
}
