// Softmax attention over a sliding window and the pooled blocks before it (see pooled_attn.cu) on the tensor cores,
// bfloat16, for prompt portions and single tokens alike.
//
// Grid (query tile, kv head, sequence).  The rows of a query tile are (token, head-in-group) pairs of one kv head,
// 128 (64 for heads above 128 values) to a block, so the query heads that share a kv head share every tile that is
// fetched.  A block walks one list of 64-entry tiles: first the tiles of the block pages that hold a block any of
// its rows may read, then the tiles of the token pages from the oldest row's window to the newest row's own key
// (cp.async, two stages).  S = Q K^T and O += P V run on m16n8k16 (bfloat16 in, float32 accumulate); scale, cap,
// masks, running maximum, denominator and output are float32.  A row at position p with lo = max(0, p - window + 1)
// reads the tokens lo .. p and the blocks 0 .. lo / P - 1.  Keys and values have sizes of their own (D, Dv).
//
// A step of single tokens has one query tile per (kv head, sequence), too few blocks for the GPU: the tile list is
// then cut into `splits` equal ranges, one block each, which leave their running maximum, denominator and
// unnormalised output in scratch; pw_attn_merge_kernel adds the ranges up in ascending order.  How many ranges
// there are depends on the batch's size alone, so a captured step replays the same launches.
#include "attn_mma.cuh"

namespace q3 {

constexpr int PWM_BN = 64;  // entries per tile

// DEC: a step whose requests bring at most 16 (token, head) rows per kv head (single tokens): one row group of 16 to
// a block, and the block's four warps take a quarter of every tile's 64 entries each, with a running maximum,
// denominator and output of their own, which meet in shared memory at the end.
template <int KT, int VT, bool DEC = false>
struct PwShape {
  static constexpr int D = 16 * KT, DV = 16 * VT;
  static constexpr int KPITCH = D + 8, VPITCH = DV + 8;
  static constexpr int KTILE = PWM_BN * KPITCH, VTILE = PWM_BN * VPITCH;
  static constexpr int WARPS = DEC ? 4 : ((KT <= 8 && VT <= 8) ? 8 : 4);
  static constexpr int BM = DEC ? 16 : 16 * WARPS;
  static constexpr int MIN_BLOCKS = DEC ? 3 : ((KT <= 8 && VT <= 8) ? 2 : 1);
  static constexpr size_t SMEM_BYTES = sizeof(__nv_bfloat16) * (size_t)(BM * KPITCH + 2 * (KTILE + VTILE));
};

// tanh through one exponential: 1 - 2 / (e^(2x) + 1); absolute error of a few 1e-7, both tails exact
__device__ __forceinline__ float pw_tanh(float x) { return 1.0f - __fdividef(2.0f, __expf(2.0f * x) + 1.0f); }

template <int KT, int VT, bool DEC>
__global__ void __launch_bounds__(PwShape<KT, VT, DEC>::WARPS * 32, PwShape<KT, VT, DEC>::MIN_BLOCKS)
pw_attn_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pages,
                   const __nv_bfloat16* __restrict__ v_pages, const __nv_bfloat16* __restrict__ pk_pages,
                   const __nv_bfloat16* __restrict__ pv_pages, __nv_bfloat16* __restrict__ out, int ldo,
                   const int* __restrict__ q_start, const int* __restrict__ kv_len, const int* __restrict__ block_table,
                   int table_stride, int num_pages, const int* __restrict__ pooled_table, int ptable_stride,
                   int num_ppages, int page_size, int Hq, int Hkv, float scale, float cap, float out_scale, int window,
                   int P, int block_limit, int splits, int T_total, float* __restrict__ part_o,
                   float* __restrict__ part_ml, int* status) {
  pdl_wait();
  pdl_launch_dependents();
  using S = PwShape<KT, VT, DEC>;
  constexpr int D = S::D, DV = S::DV, KPITCH = S::KPITCH, VPITCH = S::VPITCH, KCPR = D / 8, VCPR = DV / 8;
  constexpr int WARPS = S::WARPS, BM = S::BM;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* kv_s = q_s + BM * KPITCH;  // [stage][K tile | V tile]
  constexpr int STAGE = S::KTILE + S::VTILE;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gid = lane >> 2, tid4 = lane & 3;
  const int wrow = DEC ? 0 : warp * 16;  // the warp's first row of the block's rows
  const int qt = blockIdx.x, hk = blockIdx.y, b = blockIdx.z / splits, sp = blockIdx.z - b * splits;
  const int g = Hq / Hkv;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int len = kv_len[b];
  const int total_rows = q_len * g;
  const int row0 = qt * BM;
  if (row0 >= total_rows) return;
  const int past = len - q_len;  // position of this step's first token
  if (past < 0) {
    if (threadIdx.x == 0) atomicOr(status, Q3_STATUS_BAD_POSITION);
    return;
  }
  const int* table = block_table + (size_t)b * table_stride;
  const int* ptable = pooled_table + (size_t)b * ptable_stride;
  const int last_row = min(total_rows, row0 + BM) - 1;
  const int pos_first = past + row0 / g, pos_last = past + last_row / g;
  const int lo_key = max(0, pos_first - window + 1);
  const int blocks_hi = min(max(0, pos_last - window + 1) / P, block_limit);  // blocks the newest row reads
  const int ptiles = (blocks_hi + PWM_BN - 1) / PWM_BN;
  const int tile_lo = lo_key / PWM_BN, tile_hi = pos_last / PWM_BN;
  const int tiles = ptiles + tile_hi - tile_lo + 1;
  const int vt_begin = (int)((long long)tiles * sp / splits), vt_end = (int)((long long)tiles * (sp + 1) / splits);

  for (int e = threadIdx.x; e < BM * KCPR; e += WARPS * 32) {
    const int rr = e / KCPR, c = e % KCPR;
    const int R = row0 + rr;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (R < total_rows)
      v = *reinterpret_cast<const uint4*>(q + ((size_t)(qs + R / g) * Hq + hk * g + R % g) * D + c * 8);
    *reinterpret_cast<uint4*>(q_s + rr * KPITCH + c * 8) = v;
  }

  constexpr int LANES_PER_ROW = WARPS * 32 / PWM_BN;  // threads that share an entry: 2 or 4
  auto load_tile = [&](int vt, int stage) {
    const int row = threadIdx.x / LANES_PER_ROW, part = threadIdx.x % LANES_PER_ROW;
    const bool pooled = vt < ptiles;
    const int n = (pooled ? vt : tile_lo + vt - ptiles) * PWM_BN + row;
    const __nv_bfloat16 *ks = k_pages, *vs = v_pages;
    int bytes = 0;
    if (pooled ? n < blocks_hi : (n >= lo_key && n <= pos_last)) {
      const int page = pooled ? table_page(ptable, n / page_size, ptable_stride, status)
                              : table_page(table, n / page_size, table_stride, status);
      if (page >= 0 && page < (pooled ? num_ppages : num_pages)) {
        const size_t slot = ((size_t)page * Hkv + hk) * page_size + (n % page_size);
        ks = (pooled ? pk_pages : k_pages) + slot * D;
        vs = (pooled ? pv_pages : v_pages) + slot * DV;
        bytes = 16;
      } else {
        atomicOr(status, Q3_STATUS_BAD_PAGE);
      }
    }
    __nv_bfloat16* kd = kv_s + (size_t)stage * STAGE + row * KPITCH;
    __nv_bfloat16* vd = kv_s + (size_t)stage * STAGE + S::KTILE + row * VPITCH;
#pragma unroll
    for (int c = part; c < KCPR; c += LANES_PER_ROW) cp_async_16(kd + c * 8, ks + (bytes ? c * 8 : 0), bytes);
#pragma unroll
    for (int c = part; c < VCPR; c += LANES_PER_ROW) cp_async_16(vd + c * 8, vs + (bytes ? c * 8 : 0), bytes);
  };

  if (vt_begin < vt_end) load_tile(vt_begin, 0);
  cp_async_commit();
  __syncthreads();  // the query tile is in place

  const __nv_bfloat16* q_warp = q_s + (wrow + (lane & 7) + ((lane >> 3) & 1) * 8) * KPITCH + (lane >> 4) * 8;

  int row_pos[2], row_lo[2], row_blocks[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int R = row0 + wrow + gid + 8 * r;
    row_pos[r] = R < total_rows ? past + R / g : pos_last;  // rows past the end compute something finite, unused
    row_lo[r] = max(0, row_pos[r] - window + 1);
    row_blocks[r] = min(row_lo[r] / P, block_limit);
  }

  float o[2 * VT][4];
#pragma unroll
  for (int i = 0; i < 2 * VT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float inv_cap = cap > 0.f ? 1.0f / cap : 0.f;
  constexpr float LOG2E = 1.4426950408889634f;

  for (int vt = vt_begin; vt < vt_end; ++vt) {
    const int stage = (vt - vt_begin) & 1;
    if (vt + 1 < vt_end) load_tile(vt + 1, stage ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const __nv_bfloat16* kt_s = kv_s + (size_t)stage * STAGE;
    const __nv_bfloat16* vt_s = kt_s + S::KTILE;

    float s[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int kt = 0; kt < KT; ++kt) {
      uint32_t qf[4];
      ldmatrix_x4(qf, q_warp + kt * 16);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        if (DEC && np != warp) continue;  // this warp's sixteen entries of the tile
        uint32_t kb[4];
        ldmatrix_x4(kb, kt_s + (np * 16 + (lane & 7) + ((lane >> 4) << 3)) * KPITCH + kt * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], qf, kb[0], kb[1]);
        mma_bf16(s[2 * np + 1], qf, kb[2], kb[3]);
      }
    }
    const bool pooled = vt < ptiles;
    const int base_n = (pooled ? vt : tile_lo + vt - ptiles) * PWM_BN;
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (DEC && (nt >> 1) != warp) continue;
        const int n = base_n + nt * 8 + 2 * tid4 + (j & 1);
        float v = s[nt][j] * scale;
        if (cap > 0.f) v = cap * pw_tanh(v * inv_cap);
        v *= LOG2E;
        const int r = j >> 1;
        const bool hidden = pooled ? n >= row_blocks[r] : (n > row_pos[r] || n < row_lo[r]);
        s[nt][j] = hidden ? -INFINITY : v;
      }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float mx = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt)
        if (!DEC || (nt >> 1) == warp) mx = fmaxf(mx, fmaxf(s[nt][2 * r], s[nt][2 * r + 1]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float m_new = fmaxf(m[r], mx);
      const float m_use = m_new == -INFINITY ? 0.f : m_new;
      const float alpha = exp2f(m[r] - m_use);
      m[r] = m_new;
      l[r] *= alpha;
#pragma unroll
      for (int i = 0; i < 2 * VT; ++i) {
        o[i][2 * r] *= alpha;
        o[i][2 * r + 1] *= alpha;
      }
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        if (DEC && (nt >> 1) != warp) continue;
        const float p0 = exp2f(s[nt][2 * r] - m_use), p1 = exp2f(s[nt][2 * r + 1] - m_use);
        s[nt][2 * r] = p0;
        s[nt][2 * r + 1] = p1;
        l[r] += p0 + p1;
      }
    }
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      if (DEC && kk != warp) continue;
      uint32_t pa[4];
      pa[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      pa[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      pa[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      pa[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int dt = 0; dt < VT; ++dt) {
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, vt_s + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VPITCH + dt * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * dt], pa, vb[0], vb[1]);
        mma_bf16(o[2 * dt + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();  // this stage may be overwritten by the load issued in the next iteration
  }
  cp_async_wait<0>();

  if constexpr (DEC) {
    // the four warps' shares of the 16 rows meet in shared memory (the tiles are done with: the loop's last barrier)
    constexpr int MP = DV + 2;  // a row's output, maximum and denominator
    float* mb = reinterpret_cast<float*>(kv_s);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
      float* dst = mb + (size_t)(warp * 16 + gid + 8 * r) * MP;
      if (tid4 == 0) {
        dst[DV] = m[r];
        dst[DV + 1] = l[r];
      }
#pragma unroll
      for (int nt = 0; nt < 2 * VT; ++nt) {
        dst[nt * 8 + 2 * tid4] = o[nt][2 * r];
        dst[nt * 8 + 2 * tid4 + 1] = o[nt][2 * r + 1];
      }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 16 * DV; e += WARPS * 32) {
      const int rr = e / DV, d = e - rr * DV;
      const int R = row0 + rr;
      if (R >= total_rows) continue;
      float mx = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) mx = fmaxf(mx, mb[(size_t)(w * 16 + rr) * MP + DV]);
      float acc = 0.f, den = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float* src = mb + (size_t)(w * 16 + rr) * MP;
        if (src[DV] == -INFINITY) continue;
        const float wgt = exp2f(src[DV] - mx);
        den = fmaf(wgt, src[DV + 1], den);
        acc = fmaf(wgt, src[d], acc);
      }
      if (splits > 1) {
        const size_t row = ((size_t)sp * T_total + qs + R / g) * Hq + hk * g + R % g;
        part_o[row * DV + d] = acc;
        if (d == 0) {
          part_ml[2 * row] = mx;
          part_ml[2 * row + 1] = den;
        }
      } else {
        out[(size_t)(qs + R / g) * ldo + (size_t)(hk * g + R % g) * DV + d] =
            __float2bfloat16_rn(den > 0.f ? acc * (out_scale / den) : 0.f);
      }
    }
  } else {
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    const int R = row0 + warp * 16 + gid + 8 * r;
    if (R >= total_rows) continue;
    if (splits > 1) {  // this range's share: maximum (base-2 units), denominator, unnormalised output
      const size_t row = ((size_t)sp * T_total + qs + R / g) * Hq + hk * g + R % g;
      if (tid4 == 0) {
        part_ml[2 * row] = m[r];
        part_ml[2 * row + 1] = l[r];
      }
      float* dst = part_o + row * DV + 2 * tid4;
#pragma unroll
      for (int nt = 0; nt < 2 * VT; ++nt) *reinterpret_cast<float2*>(dst + nt * 8) = make_float2(o[nt][2 * r], o[nt][2 * r + 1]);
      continue;
    }
    const float inv = l[r] > 0.f ? out_scale / l[r] : 0.f;
    __nv_bfloat16* dst = out + (size_t)(qs + R / g) * ldo + (size_t)(hk * g + R % g) * DV + 2 * tid4;
#pragma unroll
    for (int nt = 0; nt < 2 * VT; ++nt)
      *reinterpret_cast<__nv_bfloat162*>(dst + nt * 8) = __floats2bfloat162_rn(o[nt][2 * r] * inv, o[nt][2 * r + 1] * inv);
  }
  }
}

// grid (tokens, heads), a thread per output value: the ranges' shares in ascending order.
__global__ void pw_attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                     __nv_bfloat16* __restrict__ out, int ldo, int T_total, int Hq, int DV, int splits,
                                     float out_scale) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y;
  float mx = -INFINITY;
  for (int s = 0; s < splits; ++s) mx = fmaxf(mx, part_ml[2 * (((size_t)s * T_total + t) * Hq + h)]);
  for (int d = threadIdx.x; d < DV; d += blockDim.x) {
    float acc = 0.f, den = 0.f;
    for (int s = 0; s < splits; ++s) {
      const size_t row = ((size_t)s * T_total + t) * Hq + h;
      const float ms = part_ml[2 * row];
      if (ms == -INFINITY) continue;
      const float w = exp2f(ms - mx);
      den = fmaf(w, part_ml[2 * row + 1], den);
      acc = fmaf(w, part_o[row * DV + d], acc);
    }
    out[(size_t)t * ldo + (size_t)h * DV + d] = __float2bfloat16_rn(den > 0.f ? acc * (out_scale / den) : 0.f);
  }
}

template <int KT, int VT, bool DEC>
static int pw_attn_mma_launch(const void* q, const void* k_pages, const void* v_pages, const void* pk_pages,
                              const void* pv_pages, void* out, int ldo, const int* q_start, const int* kv_len,
                              const int* table, int stride, int num_pages, const int* ptable, int pstride, int num_ppages,
                              int page_size, int B, int max_q_len, int Hq, int Hkv, float scale, float cap, float out_scale,
                              int window, int P, int block_limit, int T_total, float* part_o, float* part_ml,
                              long long part_rows, int* status, cudaStream_t stream) {
  using S = PwShape<KT, VT, DEC>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(pw_attn_mma_kernel<KT, VT, DEC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)S::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int g = Hq / Hkv;
  const long long tiles = ((long long)max_q_len * g + S::BM - 1) / S::BM;
  if (tiles > 0x7fffffffLL) return Q3_ERR_SIZE;
  // one query tile per (kv head, sequence): ranges of the keys until two blocks per SM are there, as far as the
  // scratch goes
  int splits = 1;
  if (tiles == 1 && part_o && part_ml && T_total > 0) {
    const long long blocks = (long long)Hkv * B, room = part_rows / ((long long)T_total * Hq);
    long long want = ((DEC ? 4LL : 2LL) * sm_count() + blocks - 1) / blocks;
    want = want < room ? want : room;
    splits = (int)(want < 1 ? 1 : (want > 32 ? 32 : want));
    if ((long long)B * splits > 65535) splits = 1;
  }
  q3::launch(pw_attn_mma_kernel<KT, VT, DEC>, dim3((unsigned)tiles, Hkv, B * splits), dim3(S::WARPS * 32), S::SMEM_BYTES, stream,
             (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pages, (const __nv_bfloat16*)v_pages,
             (const __nv_bfloat16*)pk_pages, (const __nv_bfloat16*)pv_pages, (__nv_bfloat16*)out, ldo, q_start, kv_len, table,
             stride, num_pages, ptable, pstride, num_ppages, page_size, Hq, Hkv, scale, cap, out_scale, window, P, block_limit,
             splits, T_total, part_o, part_ml, status);
  if (splits > 1)
    q3::launch(pw_attn_merge_kernel, dim3(T_total, Hq), dim3(S::DV < 128 ? S::DV : 128), 0, stream, (const float*)part_o,
               (const float*)part_ml, (__nv_bfloat16*)out, ldo, T_total, Hq, S::DV, splits, out_scale);
  return launch_status();
}

}  // namespace q3

// 1 if q3_pw_attn_mma has a kernel for keys of D and values of Dv values.
extern "C" int q3_pw_attn_mma_takes(int D, int Dv) {
  const bool d_ok = D == 32 || D == 64 || D == 128, v_ok = Dv == 32 || Dv == 64 || Dv == 128;
  return d_ok && v_ok ? 1 : 0;
}

// q: bf16 [T, Hq, D]; token pages k [pages, Hkv, page, D], v [.., Dv]; block pages pk, pv alike; out: rows of `ldo`
// values, head h at column h * Dv, times out_scale.  cap <= 0: no cap.  part_o (float32, part_rows * Dv values) and part_ml
// (float32, part_rows * 2 values), or null: scratch for a step of T tokens whose keys are cut into ranges (part_rows /
// (T * Hq) of them at most).  block_limit: only the first so many blocks are ever read (negative: all).
extern "C" int q3_pw_attn_mma(const void* q, const void* k_pages, const void* v_pages, const void* pk_pages,
                              const void* pv_pages, void* out, int ldo, const int* q_start, const int* kv_len,
                              const int* table, int stride, int num_pages, const int* ptable, int pstride, int num_ppages,
                              int page_size, int B, int max_q_len, int Hq, int Hkv, int D, int Dv, float scale, float cap,
                              float out_scale, int window, int P, int block_limit, int T, float* part_o, float* part_ml,
                              long long part_rows, int* status, cudaStream_t stream) {
  if (block_limit < 0) block_limit = 0x7fffffff;  // all blocks
  if (B <= 0 || max_q_len <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv || !q3_pw_attn_mma_takes(D, Dv) || page_size <= 0 || stride <= 0 || pstride <= 0 || B > 65535 ||
      Hkv > 65535 || window <= 0 || P <= 0 || ldo % 2)
    return Q3_ERR_SIZE;
  if ((uintptr_t)q % 16 || (uintptr_t)k_pages % 16 || (uintptr_t)v_pages % 16 || (uintptr_t)pk_pages % 16 ||
      (uintptr_t)pv_pages % 16 || (uintptr_t)out % 4)
    return Q3_ERR_ALIGN;
#define Q3_PW_CASE(KT, VT)                                                                                              \
  if (D == 16 * KT && Dv == 16 * VT) {                                                                                  \
    if ((long long)max_q_len * (Hq / Hkv) <= 16)                                                                        \
      return q3::pw_attn_mma_launch<KT, VT, true>(q, k_pages, v_pages, pk_pages, pv_pages, out, ldo, q_start, kv_len,   \
                                                  table, stride, num_pages, ptable, pstride, num_ppages, page_size, B,  \
                                                  max_q_len, Hq, Hkv, scale, cap, out_scale, window, P, block_limit, T, part_o, \
                                                  part_ml, part_rows, status, stream);                                  \
    return q3::pw_attn_mma_launch<KT, VT, false>(q, k_pages, v_pages, pk_pages, pv_pages, out, ldo, q_start, kv_len,    \
                                                 table, stride, num_pages, ptable, pstride, num_ppages, page_size, B,   \
                                                 max_q_len, Hq, Hkv, scale, cap, out_scale, window, P, block_limit, T, part_o, \
                                                 part_ml, part_rows, status, stream);                                   \
  }
  Q3_PW_CASE(2, 2) Q3_PW_CASE(2, 4) Q3_PW_CASE(2, 8) Q3_PW_CASE(4, 2) Q3_PW_CASE(4, 4) Q3_PW_CASE(4, 8) Q3_PW_CASE(8, 2)
  Q3_PW_CASE(8, 4) Q3_PW_CASE(8, 8)
#undef Q3_PW_CASE
  return Q3_ERR_SIZE;
}
