// Attention over cached latents on the tensor cores (bfloat16, mma.sync m16n8k16), for prompt portions and for
// single tokens.  See latent_attn.cu for the arithmetic: every head's key is the token's latent c (`rank` values)
// followed by the shared rotated part r (`rot` values), its value is c again, so one tile of keys in shared memory
// serves all heads and all tokens of a request's portion.
//
// Rows are (token, head) pairs of one request, sixteen to a row group; a row group is four warps.  Per tile of
// LM_KT keys (32, or 16 in the form for single tokens):
//   scores   the reduction over the rank + rot key values is cut into four ranges, one per warp, whose slice of
//            the queries stays in registers as A fragments for the whole kernel (a row group reads a key tile
//            once, not once per warp); the four partial score tiles meet in shared memory and every warp sums them
//            in the same order;
//   softmax  float32, every warp for the whole 16 x LM_KT tile (so no exchange of maxima), weights packed to
//            bfloat16 A fragments in registers;
//   output   the rank output columns are cut into four ranges, one per warp: O[16, rank / 4] += P V.
// Key tiles are fetched with cp.async straight out of the pages, double-buffered.  With several key ranges per
// request (single tokens over a long context) each range leaves (maximum, sum, unnormalised output) and
// latent_attn_merge adds the ranges up in a fixed order.
#include "attn_mma.cuh"

namespace q3 {


__device__ __forceinline__ float lm_exp2(float x) {  // 2^x by the hardware's unit; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// KS: k-steps of 16 per warp in the scores (rank + rot padded to 64 * KS); NO: pairs of 8-column output tiles per
// warp (rank = 64 * NO); RG: row groups per block; LM_KT: keys per tile (32 for two row groups; 16 for one, the form of
// single tokens, whose blocks are bound by the latency of their tiles: the smaller tile lets an SM hold four).
template <int KS, int NO, int RG, int LM_KT>
__global__ void __launch_bounds__(RG * 128, RG == 2 ? 2 : 4)
latent_attn_mma_kernel(const float* __restrict__ q_abs, const __nv_bfloat16* __restrict__ q_rot,
                       const __nv_bfloat16* __restrict__ c_pages, const __nv_bfloat16* __restrict__ r_pages,
                       const int* __restrict__ q_start, const int* __restrict__ kv_len, const int* __restrict__ table,
                       int stride, int page_size, int num_pages, __nv_bfloat16* __restrict__ out,
                       float* __restrict__ partial, int Ttot, int H, int rank, int rot, float scale_log2, int splits,
                       int page_shift, const float* __restrict__ sink, int* status) {
  constexpr int DKP = 64 * KS, PITCH = DKP + 8, BM = 16 * RG;
  extern __shared__ __align__(16) unsigned char lm_smem[];
  __nv_bfloat16* k_s = reinterpret_cast<__nv_bfloat16*>(lm_smem);                       // [2][LM_KT][PITCH]
  float* sp = reinterpret_cast<float*>(lm_smem + (size_t)2 * LM_KT * PITCH * sizeof(__nv_bfloat16));  // [RG][4 warps][LM_KT / 8][32 lanes] float4
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.x, split = blockIdx.z;
  const int t0 = q_start[b], q_len = q_start[b + 1] - t0;
  const int R0 = blockIdx.y * BM;
  if (R0 >= q_len * H) return;
  const int kv = kv_len[b];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int rg = warp >> 2, w = warp & 3, gid = lane >> 2, tid4 = lane & 3;
  const int rows_total = q_len * H;
  // this block's keys: everything the last of its tokens may see, cut into `splits` ranges of whole tiles
  const int last_row = min(R0 + BM, rows_total) - 1;
  const int keys = kv - q_len + last_row / H + 1;
  const int tiles_all = (keys + LM_KT - 1) / LM_KT;
  const int per = (tiles_all + splits - 1) / splits;
  const int tile_lo = split * per, tile_hi = min(tiles_all, tile_lo + per);

  // the two rows of this thread's fragments
  int row_t[2], row_h[2], row_pos[2];
  bool row_ok[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int R = R0 + rg * 16 + gid + 8 * r;
    row_ok[r] = R < rows_total;
    const int tq = row_ok[r] ? R / H : 0;
    row_t[r] = t0 + tq;
    row_h[r] = row_ok[r] ? R - tq * H : 0;
    row_pos[r] = row_ok[r] ? kv - q_len + tq : -1;
  }
  // this warp's slice of the queries: columns w * 16 KS .. of [q_abs | q_rot | zeros]
  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = i & 1, d = (w * KS + ks) * 16 + 2 * tid4 + (i >> 1) * 8;
      float v0 = 0.f, v1 = 0.f;
      if (row_ok[r]) {
        if (d < rank) {
          const float2 v = *reinterpret_cast<const float2*>(q_abs + ((size_t)row_h[r] * Ttot + row_t[r]) * rank + d);
          v0 = v.x;
          v1 = v.y;
        } else if (d < rank + rot) {
          const __nv_bfloat162 v =
              *reinterpret_cast<const __nv_bfloat162*>(q_rot + ((size_t)row_t[r] * H + row_h[r]) * rot + (d - rank));
          v0 = __low2float(v);
          v1 = __high2float(v);
        }
      }
      qa[ks][i] = pack_bf16(v0, v1);
    }

  const int* trow = table + (size_t)b * stride;
  // LM_KT keys by RG * 128 threads: a key's row is copied by TPK threads, which look its page up once
  constexpr int TPK = RG * 128 / LM_KT, CHUNKS = DKP / 8;
  const int load_j = threadIdx.x / TPK, load_c = threadIdx.x % TPK;
  // the page of this thread's key in a tile (-1: a hole or a bad id, -2: past the block's keys); asked for one tile
  // before the copy that needs it, so that the table's answer is there when the copy is issued
  auto page_of = [&](int tile) {
    const int n = tile * LM_KT + load_j;
    return n < keys ? table_page(trow, page_shift >= 0 ? n >> page_shift : n / page_size, stride, status) : -2;
  };
  auto load_tile = [&](int tile, int stage, int page) {
    __nv_bfloat16* dst = k_s + ((size_t)stage * LM_KT + load_j) * PITCH;
    const int n = tile * LM_KT + load_j;
    const __nv_bfloat16* c_src = c_pages;
    const __nv_bfloat16* r_src = r_pages;
    bool ok = false;
    if (page >= 0 && page < num_pages) {
      const size_t slot = (size_t)page * page_size + (page_shift >= 0 ? n & (page_size - 1) : n % page_size);
      c_src = c_pages + slot * rank;
      r_src = r_pages + slot * rot;
      ok = true;
    } else if (page != -2 && load_c == 0) {
      atomicOr(status, Q3_STATUS_BAD_PAGE);
    }
#pragma unroll
    for (int c = load_c; c < CHUNKS; c += TPK) {
      const int d = c * 8;
      const bool real = ok && d < rank + rot;
      cp_async_16(dst + d, real ? (d < rank ? c_src + d : r_src + (d - rank)) : c_pages, real ? 16 : 0);
    }
  };

  float o[2 * NO][4];
#pragma unroll
  for (int i = 0; i < 2 * NO; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

  if (tile_lo < tile_hi) load_tile(tile_lo, 0, page_of(tile_lo));
  cp_async_commit();
  int page_next = tile_lo + 1 < tile_hi ? page_of(tile_lo + 1) : -2;
  for (int tile = tile_lo; tile < tile_hi; ++tile) {
    const int stage = (tile - tile_lo) & 1;
    if (tile + 1 < tile_hi) load_tile(tile + 1, stage ^ 1, page_next);
    if (tile + 2 < tile_hi) page_next = page_of(tile + 2);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* kt_s = k_s + (size_t)stage * LM_KT * PITCH;

    // partial scores over this warp's range of the reduction
    float s[LM_KT / 8][4];
#pragma unroll
    for (int i = 0; i < LM_KT / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int np = 0; np < LM_KT / 16; ++np) {
        uint32_t kb[4];
        ldmatrix_x4(kb, kt_s + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * PITCH + (w * KS + ks) * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], qa[ks], kb[0], kb[1]);
        mma_bf16(s[2 * np + 1], qa[ks], kb[2], kb[3]);
      }
    }
    // the four warps of a row group hold the same places of the tile in the same lanes: a lane leaves its fragment
    // as whole float4s, [warp][n-tile][lane], and reads the other warps' at its own lane
    float4* sp4 = reinterpret_cast<float4*>(sp) + (size_t)rg * 4 * (LM_KT / 8) * 32;
#pragma unroll
    for (int nt = 0; nt < LM_KT / 8; ++nt)
      sp4[(w * (LM_KT / 8) + nt) * 32 + lane] = make_float4(s[nt][0], s[nt][1], s[nt][2], s[nt][3]);
    __syncthreads();
    // the whole tile's scores, summed in the order of the warps
    const int base_n = tile * LM_KT;
#pragma unroll
    for (int nt = 0; nt < LM_KT / 8; ++nt) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int ww = 0; ww < 4; ++ww) {
        const float4 v = sp4[(ww * (LM_KT / 8) + nt) * 32 + lane];
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
      }
      const int n = base_n + nt * 8 + 2 * tid4;
      s[nt][0] = n <= row_pos[0] ? acc.x * scale_log2 : -INFINITY;
      s[nt][1] = n + 1 <= row_pos[0] ? acc.y * scale_log2 : -INFINITY;
      s[nt][2] = n <= row_pos[1] ? acc.z * scale_log2 : -INFINITY;
      s[nt][3] = n + 1 <= row_pos[1] ? acc.w * scale_log2 : -INFINITY;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < LM_KT / 8; ++nt) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[r], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = lm_exp2(m[r] - m_use);
      const bool grew = m_new != m[r];
      m[r] = m_new;
      l[r] *= alpha;
      if (__any_sync(0xffffffffu, grew)) {  // most tiles leave every row's maximum where it was
#pragma unroll
        for (int i = 0; i < 2 * NO; ++i) {
          o[i][2 * r] *= alpha;
          o[i][2 * r + 1] *= alpha;
        }
      }
#pragma unroll
      for (int nt = 0; nt < LM_KT / 8; ++nt) {
        const float p0 = lm_exp2(s[nt][2 * r] - m_use), p1 = lm_exp2(s[nt][2 * r + 1] - m_use);
        s[nt][2 * r] = p0;
        s[nt][2 * r + 1] = p1;
        l[r] += p0 + p1;
      }
    }
    // O[:, this warp's columns] += P V, V = the tile's latents
#pragma unroll
    for (int kk = 0; kk < LM_KT / 16; ++kk) {
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dt = 0; dt < NO; ++dt) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, kt_s + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * PITCH + (w * NO + dt) * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
        mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();  // the stage and the score tiles may be written again
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    if (!row_ok[r]) continue;
    const size_t row = (size_t)row_t[r] * H + row_h[r];
    if (splits == 1) {
      float keep = 1.f;
      if (sink) {  // one more term in the denominator: exp(sink), in the base-2 scale of the scores
        const float s2 = sink[row_h[r]] * 1.4426950408889634f, m_new = fmaxf(m[r], s2);
        keep = lm_exp2(m[r] - m_new);
        l[r] = fmaf(l[r], keep, lm_exp2(s2 - m_new));
      }
      const float inv = l[r] > 0.f ? keep / l[r] : 0.f;
      __nv_bfloat16* dst = out + row * rank + w * NO * 16 + 2 * tid4;
#pragma unroll
      for (int i = 0; i < 2 * NO; ++i)
        *reinterpret_cast<__nv_bfloat162*>(dst + i * 8) = __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
    } else {
      float* dst = partial + (row * splits + split) * (rank + 2);
      if (w == 0 && tid4 == 0) {
        dst[0] = m[r];
        dst[1] = l[r];
      }
#pragma unroll
      for (int i = 0; i < 2 * NO; ++i)
        *reinterpret_cast<float2*>(dst + 2 + w * NO * 16 + i * 8 + 2 * tid4) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
    }
  }
}

// One block per (token, head): the key ranges' partial results added up in the order of the ranges.  A range's
// weight, 2^(its maximum - the row's maximum) / the row's sum, is worked out once per block.
constexpr int LM_MAX_SPLITS = 64;

__global__ void latent_attn_merge_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int rank,
                                         int splits, const float* __restrict__ sink, int H) {
  __shared__ float weight[LM_MAX_SPLITS];
  pdl_wait();
  pdl_launch_dependents();
  const size_t row = blockIdx.x;
  const float* p = partial + row * splits * (rank + 2);
  if (threadIdx.x < 32) {
    float mx = -INFINITY;
    for (int s = threadIdx.x; s < splits; s += 32) mx = fmaxf(mx, p[(size_t)s * (rank + 2)]);
    mx = warp_max(mx);
    const float s2 = sink ? sink[row % H] * 1.4426950408889634f : -INFINITY;  // the sink, a range without keys
    mx = fmaxf(mx, s2);
    float total = sink ? lm_exp2(s2 - mx) : 0.f;  // every lane adds all ranges in their order: the same sum in every lane
    for (int s = 0; s < splits; ++s) {
      const float ms = p[(size_t)s * (rank + 2)];
      if (ms != -INFINITY) total += p[(size_t)s * (rank + 2) + 1] * lm_exp2(ms - mx);
    }
    const float inv = total > 0.f ? 1.0f / total : 0.f;
    for (int s = threadIdx.x; s < splits; s += 32) {
      const float ms = p[(size_t)s * (rank + 2)];
      weight[s] = ms != -INFINITY ? lm_exp2(ms - mx) * inv : 0.f;
    }
  }
  __syncthreads();
  for (int d = threadIdx.x; d < rank; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc = fmaf(p[(size_t)s * (rank + 2) + 2 + d], weight[s], acc);
    out[row * rank + d] = __float2bfloat16_rn(acc);
  }
}

template <int KS, int NO, int RG>
static int lm_launch(const float* q_abs, const void* q_rot, const void* c_pages, const void* r_pages, const int* q_start,
                     const int* kv_len, const int* table, int stride, int page_size, int num_pages, void* out,
                     float* partial, int T, int B, int max_q_len, int H, int rank, int rot, float scale, int splits,
                     const float* sink, int* status, cudaStream_t stream) {
  using bf16 = __nv_bfloat16;
  constexpr int PITCH = 64 * KS + 8, LM_KT = RG == 2 ? 32 : 16;
  const size_t smem = (size_t)2 * LM_KT * PITCH * sizeof(bf16) + (size_t)RG * 4 * 16 * LM_KT * sizeof(float);
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(latent_attn_mma_kernel<KS, NO, RG, RG == 2 ? 32 : 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    configured = true;
  }
  const long long tiles = ((long long)max_q_len * H + 16 * RG - 1) / (16 * RG);
  if (tiles > 65535 || splits > LM_MAX_SPLITS) return Q3_ERR_SIZE;
  launch(latent_attn_mma_kernel<KS, NO, RG, RG == 2 ? 32 : 16>, dim3(B, (unsigned)tiles, splits), dim3(RG * 128), smem, stream, q_abs,
         (const bf16*)q_rot, (const bf16*)c_pages, (const bf16*)r_pages, q_start, kv_len, table, stride, page_size,
         num_pages, (bf16*)out, partial, T, H, rank, rot, scale * 1.4426950408889634f, splits, page_shift_of(page_size),
         sink, status);
  if (splits > 1) {
    g_launch_early = false;  // started after every range has left its result
    launch(latent_attn_merge_kernel, dim3((unsigned)((size_t)T * H)), dim3(128), 0, stream, (const float*)partial,
           (bf16*)out, rank, splits, sink, H);
    g_launch_early = true;
  }
  return launch_status();
}

}  // namespace q3

// 1 if the tensor-core kernel takes these sizes (bfloat16 only): a latent of 64, 128, 256 or 512 values and a
// rotated part in multiples of 8 that fits the padded reduction.
extern "C" int q3_latent_attn_mma_takes(int rank, int rot) {
  if (rot < 0 || rot % 8) return 0;
  const int dk = rank + rot;
  if (rank == 512) return dk <= 576;
  if (rank == 256) return dk <= 320;
  if (rank == 128) return dk <= 192;
  if (rank == 64) return dk <= 128;
  return 0;
}

// q_abs: float32 [H, T, rank]; q_rot: bf16 [T, H, rot]; pages bf16; out: bf16 [T, H * rank].  `splits` key ranges per
// request (1: the result is written at once; more: `partial` holds T * H * splits * (rank + 2) floats).  Every
// request of the step reads the keys up to each of its tokens' positions (kv_len - q_len + index).
extern "C" int q3_latent_attn_mma(const float* q_abs, const void* q_rot, const void* c_pages, const void* r_pages,
                                  const int* q_start, const int* kv_len, const int* table, int stride, int page_size,
                                  int num_pages, void* out, float* partial, int T, int B, int max_q_len, int H, int rank,
                                  int rot, float scale, int splits, const float* sink, int* status, cudaStream_t stream) {
  if (T <= 0 || B <= 0) return 0;
  if (!q3_latent_attn_mma_takes(rank, rot) || H <= 0 || max_q_len <= 0 || page_size <= 0 || stride <= 0 || splits < 1)
    return Q3_ERR_SIZE;
  if (splits > 1 && !partial) return Q3_ERR_SCRATCH;
  if ((uintptr_t)q_abs % 8 || (uintptr_t)q_rot % 4 || (uintptr_t)c_pages % 16 || (uintptr_t)r_pages % 16 ||
      (uintptr_t)out % 4)
    return Q3_ERR_ALIGN;
  const bool wide = (long long)max_q_len * H > 16;  // more than one row group's rows per request
#define Q3_LM(KS, NO)                                                                                                  \
  return wide ? q3::lm_launch<KS, NO, 2>(q_abs, q_rot, c_pages, r_pages, q_start, kv_len, table, stride, page_size,    \
                                         num_pages, out, partial, T, B, max_q_len, H, rank, rot, scale, splits, sink,  \
                                         status, stream)                                                               \
              : q3::lm_launch<KS, NO, 1>(q_abs, q_rot, c_pages, r_pages, q_start, kv_len, table, stride, page_size,    \
                                         num_pages, out, partial, T, B, max_q_len, H, rank, rot, scale, splits, sink,  \
                                         status, stream);
  if (rank == 512) { Q3_LM(9, 8) }
  if (rank == 256) { Q3_LM(5, 4) }
  if (rank == 128) { Q3_LM(3, 2) }
  Q3_LM(2, 1)
#undef Q3_LM
}
