// Routed experts for many tokens on the fifth-generation tensor cores (bfloat16): the (token, expert) pairs of a step
// are sorted by expert, every expert's rows padded to whole tiles of 128, and both products of all experts run as one
// grouped product each, C[rows of tile m] = A[rows of tile m] * W[expert of tile m]^T.
//
//   moe_sort        one block: counts the pairs of every expert, lays the experts out one after the other in whole
//                   tiles, and gives every pair its row.  Leaves pos[pair] (the pair's row, -1 for an expert id out
//                   of range), src[row] (the row's pair, -1 for padding) and meta = {tiles in use, expert of tile 0,
//                   expert of tile 1, ...}.  Which row of its expert a pair gets is not fixed from run to run; a
//                   row's product does not depend on where in a tile it lies.
//   moe_gather      row r of the sorted input = the token's row of h (zeros for padding), times the pair's router
//                   weight where that weight belongs to what the expert reads (`in_wts`).
//   moe_grouped     the persistent kernel of gemm_tc.cu (TMA loader, one tcgen05.mma thread, accumulators in tensor
//                   memory, epilogue warps) over the tiles that `meta` lists: the tile's rows of W start at
//                   expert * N.  The number of tiles is read on the device, so a step's launches do not depend on
//                   the routing and a captured graph replays them.  The epilogue applies the activation; for gated
//                   experts (gate and up rows alternating in blocks of 16 rows of a stack of 2 F) it multiplies the
//                   activated gate columns of a 32-column piece by the piece's up columns and stores 16 values.
//   moe_combine     out[t] = base[t] + sum_k weight[t, k] y[pos[t, k]], float32 sums in the router's order.
//
// Every wait on an mbarrier is bounded as in gemm_tc.cu: a wait that runs out sets the TIMEOUT bit of the status word,
// every role leaves its loop, tensor memory is released and the block returns.
#include "tc_common.cuh"

namespace q3 {

constexpr int MOE_BM = 128;
constexpr int MOE_EPI_WARPS = 8;
constexpr int MOE_THREADS = 64 + 32 * MOE_EPI_WARPS;

template <int BN>
struct MoeShape {
  static constexpr int A_BYTES = MOE_BM * TC_BK * 2;
  static constexpr int B_BYTES = BN * TC_BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int BAR_BYTES = 256;
  static constexpr int STAGES = (192 * 1024) / STAGE_BYTES;  // 4 stages of 48 KB or 6 of 32 KB
  static constexpr size_t SMEM_BYTES = (size_t)STAGES * STAGE_BYTES + BAR_BYTES;
  static constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators
};

__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, int pairs, int E, int* __restrict__ pos, int* __restrict__ src,
                int* __restrict__ meta, int max_tiles) {
  extern __shared__ int sh[];  // [E] counts, later cursors; [E] first rows
  __shared__ int tiles_used;
  pdl_wait();
  pdl_launch_dependents();
  int* count = sh;
  int* first = sh + E;
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int tiles = 0;
    for (int e = 0; e < E; ++e) {
      first[e] = tiles * MOE_BM;
      const int n = (count[e] + MOE_BM - 1) / MOE_BM;
      for (int i = 0; i < n && tiles + i < max_tiles; ++i) meta[1 + tiles + i] = e;
      tiles += n;
      count[e] = 0;
    }
    tiles_used = min(tiles, max_tiles);  // never more than max_tiles: sum of ceil(c_e / 128) <= pairs / 128 + E
    meta[0] = tiles_used;
  }
  __syncthreads();
  const int rows = tiles_used * MOE_BM;
  for (int r = threadIdx.x; r < rows; r += blockDim.x) src[r] = -1;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int e = ids[p];
    int r = -1;
    if (e >= 0 && e < E) {
      r = first[e] + atomicAdd(&count[e], 1);
      if (r < rows) src[r] = p; else r = -1;
    }
    pos[p] = r;
  }
}

// grid (rows): eight values per thread and turn.  W a multiple of 8, rows 16-byte aligned.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ h, const int* __restrict__ src,
                                  const int* __restrict__ meta, __nv_bfloat16* __restrict__ sorted, int W, int top,
                                  const float* __restrict__ in_wts) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  if (r >= meta[0] * MOE_BM) return;
  const int p = src[r];
  const uint4* from = p >= 0 ? reinterpret_cast<const uint4*>(h + (size_t)(p / top) * W) : nullptr;
  uint4* to = reinterpret_cast<uint4*>(sorted + (size_t)r * W);
  if (!from || !in_wts) {
    for (int i = threadIdx.x; i < W / 8; i += blockDim.x) to[i] = from ? from[i] : make_uint4(0, 0, 0, 0);
    return;
  }
  const float w = in_wts[p];  // the expert reads the row times its weight, rounded once
  for (int i = threadIdx.x; i < W / 8; i += blockDim.x) {
    uint4 v = from[i];
    __nv_bfloat162* v2 = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(v2[j]);
      v2[j] = __floats2bfloat162_rn(f.x * w, f.y * w);
    }
    to[i] = v;
  }
}

// grid (tokens).  y: the sorted rows of the second product.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                                   const float* __restrict__ wts, const __nv_bfloat16* __restrict__ base,
                                   __nv_bfloat16* __restrict__ out, int W, int top) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < W / 8; i += blockDim.x) {
    float acc[8];
    if (base) {
      const uint4 b = reinterpret_cast<const uint4*>(base + (size_t)t * W)[i];
      const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(b2[j]);
        acc[2 * j] = f.x;
        acc[2 * j + 1] = f.y;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    }
    for (int k = 0; k < top; ++k) {
      const int r = pos[(size_t)t * top + k];
      if (r < 0) continue;
      const float w = wts[(size_t)t * top + k];
      const uint4 v = reinterpret_cast<const uint4*>(y + (size_t)r * W)[i];
      const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(v2[j]);
        acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
        acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
    reinterpret_cast<uint4*>(out + (size_t)t * W)[i] = o;
  }
}

constexpr int MOE_GATED = 0x100;  // OR-ed into the activation code: the columns are gate and up in blocks of 16

// 32 columns of one row: activation, rounding to bfloat16, store.
__device__ __forceinline__ void moe_store_chunk(const uint32_t (&v)[32], __nv_bfloat16* C, int row, int col0, int N, int ldc,
                                                int act) {
  if (act & MOE_GATED) {  // columns col0 .. +15: gates, +16 .. +31: their up values; N = 2 ldc-columns, whole pieces
    if (col0 + 32 > N) return;
    __nv_bfloat16* dst = C + (size_t)row * ldc + (col0 >> 1);
    float g[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) g[j] = activate(__uint_as_float(v[j]), act & 0xff) * __uint_as_float(v[16 + j]);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint4 pk;
      pk.x = pack2(__float_as_uint(g[8 * j + 0]), __float_as_uint(g[8 * j + 1]));
      pk.y = pack2(__float_as_uint(g[8 * j + 2]), __float_as_uint(g[8 * j + 3]));
      pk.z = pack2(__float_as_uint(g[8 * j + 4]), __float_as_uint(g[8 * j + 5]));
      pk.w = pack2(__float_as_uint(g[8 * j + 6]), __float_as_uint(g[8 * j + 7]));
      reinterpret_cast<uint4*>(dst)[j] = pk;
    }
    return;
  }
  __nv_bfloat16* dst = C + (size_t)row * ldc + col0;
  float r[32];
#pragma unroll
  for (int j = 0; j < 32; ++j) r[j] = activate(__uint_as_float(v[j]), act);
  if (col0 + 32 <= N && ((uintptr_t)dst & 15) == 0) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 pk;
      pk.x = pack2(__float_as_uint(r[8 * j + 0]), __float_as_uint(r[8 * j + 1]));
      pk.y = pack2(__float_as_uint(r[8 * j + 2]), __float_as_uint(r[8 * j + 3]));
      pk.z = pack2(__float_as_uint(r[8 * j + 4]), __float_as_uint(r[8 * j + 5]));
      pk.w = pack2(__float_as_uint(r[8 * j + 6]), __float_as_uint(r[8 * j + 7]));
      reinterpret_cast<uint4*>(dst)[j] = pk;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < N) dst[j] = __float2bfloat16_rn(r[j]);
  }
}

// C[rows of tile m, N] = act(A[rows of tile m, K] * W[meta[1 + m] * N .., K]^T) for the meta[0] tiles in use.
template <int BN>
__global__ void __launch_bounds__(MOE_THREADS)
moe_grouped_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   __nv_bfloat16* __restrict__ C, const int* __restrict__ meta, int max_tiles, int N, int K, int E, int ldc,
                   int act, int* status) {
  using S = MoeShape<BN>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  unsigned char* tiles = smem_raw;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + (size_t)S::STAGES * S::STAGE_BYTES);
  uint64_t* empty = full + S::STAGES;
  uint64_t* acc_full = empty + S::STAGES;  // [2]
  uint64_t* acc_empty = acc_full + 2;      // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  __shared__ int abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_tiles = (K + TC_BK - 1) / TC_BK;
  const int n_tiles = (N + BN - 1) / BN;
  const bool aligned = (s_addr(smem_raw) & 1023u) == 0;
  if (!aligned && threadIdx.x == 0) atomicOr(status, Q3_STATUS_TIMEOUT);

  if (warp == 0 && lane == 0) {
    tma_prefetch_map(&map_a);
    tma_prefetch_map(&map_b);
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], MOE_EPI_WARPS);  // one arrival from each epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();  // the tile list and the rows come from the kernels before this one
  pdl_launch_dependents();
  const int m_tiles = aligned ? min(max(meta[0], 0), max_tiles) : 0;
  const int num_tiles = m_tiles * n_tiles;
  // Tensor memory is taken only after the wait (see gemm_tc.cu).
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s_addr(tmem_holder)),
                 "r"(S::TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      // ---- loader
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int mt = tile % m_tiles;
        const int e = min(max(meta[1 + mt], 0), E - 1);
        const int m0 = mt * MOE_BM, w0 = e * N + (tile / m_tiles) * BN;
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % S::STAGES;
          const uint32_t use = it / S::STAGES;
          unsigned char* a_s = tiles + (size_t)s * S::STAGE_BYTES;
          if (use > 0 && !mbar_wait(&empty[s], (use & 1) ^ 1, &abort_flag)) {
            abort_flag = 1;
            atomicOr(status, Q3_STATUS_TIMEOUT);
            ok = false;
            break;
          }
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          tma_load_2d(a_s + S::A_BYTES, &map_b, &full[s], kt * TC_BK, w0);
          tma_load_2d(a_s, &map_a, &full[s], kt * TC_BK, m0);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---- tensor-core issue
      constexpr uint32_t idesc = umma_idesc(BN);
      uint32_t it = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
        const uint32_t buf = t & 1;
        if (t >= 2 && !mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, &abort_flag)) {
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kt = 0; kt < k_tiles; ++kt, ++it) {
          const int s = it % S::STAGES;
          const uint32_t use = it / S::STAGES;
          if (!mbar_wait(&full[s], use & 1, &abort_flag)) {
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const unsigned char* a_s = tiles + (size_t)s * S::STAGE_BYTES;
          const uint64_t a_desc = umma_desc_sw128(a_s), b_desc = umma_desc_sw128(a_s + S::A_BYTES);
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k)  // 16 values of k = 32 bytes further along the swizzled row
            umma_f16(tmem_acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kt | k) != 0);
          umma_commit(&empty[s]);  // the stage is free once these instructions have read it
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
      if (!ok) {
        abort_flag = 1;
        atomicOr(status, Q3_STATUS_TIMEOUT);
      }
    }
  } else {
    // ---- epilogue: a warp may read the 32 TMEM lanes of its quarter (warp index modulo 4)
    const int quarter = warp & 3;
    uint32_t t = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++t) {
      const int m0 = (tile % m_tiles) * MOE_BM, n0 = (tile / m_tiles) * BN;
      const uint32_t buf = t & 1;
      const bool ready = mbar_wait(&acc_full[buf], (t >> 1) & 1, &abort_flag);
      if (!__all_sync(0xffffffffu, ready)) {
        if (lane == 0) {
          abort_flag = 1;
          atomicOr(status, Q3_STATUS_TIMEOUT);
        }
        ok = false;
        break;
      }
      tcgen05_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t tmem_acc = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int c0 = ((warp - 2) >> 2) * 32; c0 < BN; c0 += (MOE_EPI_WARPS / 4) * 32) {
        if (n0 + c0 >= N) break;  // uniform over the warp
        uint32_t v[32];
        tmem_ld_32(tmem_acc + (uint32_t)c0, v);
        tmem_wait_ld();
        moe_store_chunk(v, C, row, n0 + c0, N, ldc, act);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[buf]);
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(S::TMEM_COLS) : "memory");
  }
}

template <int BN>
static int moe_grouped_launch(const void* A, const void* W, void* C, const int* meta, int map_tiles, int max_tiles, int N,
                              int K, int E, int ldc, int act, int* status, cudaStream_t stream) {
  using S = MoeShape<BN>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(moe_grouped_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)S::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap map_a, map_b;
  int code = cached_map(&map_a, A, (uint64_t)map_tiles * MOE_BM, (uint64_t)K, MOE_BM);
  if (code) return code;
  code = cached_map(&map_b, W, (uint64_t)E * N, (uint64_t)K, BN);
  if (code) return code;
  const long long tiles = (long long)((N + BN - 1) / BN) * max_tiles;
  if (tiles > 0x7fffffffLL) return Q3_ERR_SIZE;
  const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
  q3::launch(moe_grouped_kernel<BN>, dim3(grid), dim3(MOE_THREADS), S::SMEM_BYTES, stream, map_a, map_b, (__nv_bfloat16*)C,
             meta, max_tiles, N, K, E, ldc, act, status);
  return launch_status();
}

}  // namespace q3

// Rows per tile of the sorted layout: every expert's rows start on a multiple of this.
extern "C" int q3_moe_tile_rows() { return q3::MOE_BM; }

// The routed experts of T tokens (bfloat16) by sorted rows and two grouped products.  h: [T, W]; up: [E, F, W];
// (gated: [E, 2 F, W], gate and up rows alternating in blocks of 16, F a multiple of 16); in_wts: [T, top] or null, the
// weights of what the experts read (`wts` are those of what they return);
// down: [E, W, F]; ids, wts: [T, top]; base: [T, W] or null; out: [T, W].  Scratch for max_tiles >= T * top / 128 + E
// tiles: sorted_in [max_tiles * 128, W], sorted_act [.., F], sorted_out [.., W], pos int32 [T * top], src int32
// [max_tiles * 128], meta int32 [1 + max_tiles].  W and F multiples of 8, all bases 16-byte aligned.
extern "C" int q3_moe_grouped(const void* h, const void* up, const void* down, const int* ids, const float* wts,
                              const void* base, void* out, void* sorted_in, void* sorted_act, void* sorted_out, int* pos,
                              int* src, int* meta, int T, int W, int F, int E, int top, int max_tiles, int act, int gated,
                              const float* in_wts, int* status, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (gated && F % 16) return Q3_ERR_SIZE;
  if (W <= 0 || F <= 0 || E <= 0 || E > 4096 || top <= 0 || W % 8 || F % 8 || (long long)T * top > 0x3fffffffll ||
      max_tiles < (int)(((long long)T * top) / q3::MOE_BM) + E || (long long)E * (W > 2 * F ? W : 2 * F) > 0x7fffffffll ||
      act < 0 || act > Q3_ACT_RELU_SQ)
    return Q3_ERR_SIZE;
  if ((uintptr_t)h % 16 || (uintptr_t)up % 16 || (uintptr_t)down % 16 || (uintptr_t)out % 16 || (uintptr_t)sorted_in % 16 ||
      (uintptr_t)sorted_act % 16 || (uintptr_t)sorted_out % 16 || (base && (uintptr_t)base % 16))
    return Q3_ERR_ALIGN;
  using bf16 = __nv_bfloat16;
  const int pairs = T * top;
  const int map_tiles = max_tiles;  // the tensor maps cover all of the scratch rows, whatever the step's size
  max_tiles = pairs / q3::MOE_BM + E;  // what this step's pairs can fill at most
  q3::launch(q3::moe_sort_kernel, dim3(1), dim3(1024), (size_t)2 * E * sizeof(int), stream, ids, pairs, E, pos, src, meta,
             max_tiles);
  q3::launch(q3::moe_gather_kernel, dim3(max_tiles * q3::MOE_BM), dim3(128), 0, stream, (const bf16*)h, (const int*)src,
             (const int*)meta, (bf16*)sorted_in, W, top, in_wts);
  int code = q3::launch_status();
  if (code) return code;
  // the tile width that needs fewer rounds of the SMs for the tiles to expect (half of the padding tiles in use)
  const long long sms = q3::sm_count();
  const long long expect = (long long)pairs / q3::MOE_BM + (E + 1) / 2;
  auto wide = [&](int n) {
    const long long t256 = expect * ((n + 255) / 256), t128 = expect * ((n + 127) / 128);
    return ((t256 + sms - 1) / sms) * 256 <= ((t128 + sms - 1) / sms) * 128;
  };
  auto product = [&](const void* a, const void* wgt, void* c, int n, int k, int ldc, int activation) {
    return wide(n) ? q3::moe_grouped_launch<256>(a, wgt, c, meta, map_tiles, max_tiles, n, k, E, ldc, activation, status, stream)
                   : q3::moe_grouped_launch<128>(a, wgt, c, meta, map_tiles, max_tiles, n, k, E, ldc, activation, status, stream);
  };
  code = gated ? product(sorted_in, up, sorted_act, 2 * F, W, F, act | q3::MOE_GATED)
               : product(sorted_in, up, sorted_act, F, W, F, act);
  if (code) return code;
  code = product(sorted_act, down, sorted_out, W, F, W, Q3_ACT_NONE);
  if (code) return code;
  q3::launch(q3::moe_combine_kernel, dim3(T), dim3(128), 0, stream, (const bf16*)sorted_out, (const int*)pos, wts,
             (const bf16*)base, (bf16*)out, W, top);
  return q3::launch_status();
}
