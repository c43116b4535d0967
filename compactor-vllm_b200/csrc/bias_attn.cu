// Attention over the paged cache with a linear distance bias, a chunk mask and an optional softmax sink,
// for any head size and 32-bit or 16-bit storage.  Three launches per layer:
//   cvllm_qknorm_store    per-head RMS norm of q and k, k and v written to their cache rows
//   cvllm_bias_attn_varlen  portions of prompts (any number of new tokens per sequence) against the cache
//   cvllm_bias_attn_decode  one new token per sequence
// score(i, j) = scale * q_i . k_j - slope_h * (i - j) for keys j <= i of the same chunk
// (floor(i / chunk) == floor(j / chunk), chunk 0 = one chunk), positions counted from the start of the
// sequence; p_j = exp(s_j) / (sink + sum_j exp(s_j)) with sink = 1 (a key of score 0 without a value) or 0.
// The new tokens' keys are in the cache before the attention launches read it, so both read keys from one place.
// All arithmetic is fp32; 16-bit storage only rounds q, k, v and the output.
#include "common.cuh"
#include "mma.cuh"

namespace cvllm {
namespace {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

struct PagedKV {
  const void* k;            // [rows, D]
  const void* v;            // [rows, Dv]
  const int32_t* table;     // [slots, G, P]
  int64_t table_stride_slot, table_stride_head;
  int page_size;
  int page_shift;           // log2(page_size) when that is a power of two, else -1
  int64_t v_stride;         // elements between value rows (Dv, or more when the values are columns of wider rows)
};

inline PagedKV make_paged(const void* k, const void* v, const int32_t* table, int64_t stride_slot, int64_t stride_head,
                          int page_size, int64_t v_stride) {
  int shift = -1;
  if ((page_size & (page_size - 1)) == 0)
    for (shift = 0; (1 << shift) < page_size; ++shift) {}
  return PagedKV{k, v, table, stride_slot, stride_head, page_size, shift, v_stride};
}

// A sliding window and a learned bias per distance, beside the linear bias and the chunk mask (all may be combined):
// a query at position i sees the keys at distances 0 .. window - 1 (window 0: no limit), and the score of the key at
// distance n gets table[min(n, rows - 1), h] (fp32 [rows, H]; NULL: none).  The table is made by the caller, so any
// rule from distance to bias (buckets of a smaller learned table, for one) is served.
struct DistBias {
  const float* table;
  int rows;
  int window;
};

__device__ __forceinline__ float dist_bias_at(const DistBias& db, int n, int H, int h) {
  return db.table ? db.table[(int64_t)min(n, db.rows - 1) * H + h] : 0.f;
}

// first position a query at position pi sees
__device__ __forceinline__ int first_key(int pi, int chunk, const DistBias& db) {
  int lo = chunk > 0 ? (pi / chunk) * chunk : 0;
  if (db.window > 0) lo = max(lo, pi - db.window + 1);
  return lo;
}

__device__ __forceinline__ int64_t cache_row(const PagedKV& c, int slot, int g, int pos) {
  const int lp = c.page_shift >= 0 ? pos >> c.page_shift : pos / c.page_size;
  const int page = c.table[slot * c.table_stride_slot + g * c.table_stride_head + lp];
  return (int64_t)page * c.page_size + (pos - lp * c.page_size);
}

// ---------------------------------------------------------------------------------------------------------
// q / k rotation + norm + store.  One CTA per token; its warps take the token's H + 2G head rows in turn.
// Rotation (inv_freq != NULL): neighbours (2i, 2i + 1) of the first rot_dims numbers of every q and k head turn by
// pos * inv_freq[i] (64-bit angle, fp32 sine / cosine in shared memory, once per CTA) BEFORE the norm.
// norm 0: no norm; 1: x / sqrt(mean(x^2) + eps), times the weight when one is given.
// ---------------------------------------------------------------------------------------------------------
struct Rotation {
  const double* inv_freq;   // [dims / 2] or NULL (no rotation)
  int dims;                 // even, <= D
};

// cos / sin of pos * inv_freq[i], i < dims / 2, into shared memory; the caller synchronises
__device__ __forceinline__ void fill_rotation(float* cs, float* sn, const Rotation& rot, int pos) {
  for (int i = threadIdx.x; i < rot.dims / 2; i += blockDim.x) {
    double sv, cv;
    sincos((double)pos * rot.inv_freq[i], &sv, &cv);
    cs[i] = (float)cv;
    sn[i] = (float)sv;
  }
}

template <typename T>
__global__ void __launch_bounds__(128) qknorm_store_kernel(
    const T* __restrict__ qkv, int64_t qkv_stride, const float* __restrict__ q_w, const float* __restrict__ k_w,
    float eps, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_slot, T* __restrict__ q_out,
    T* __restrict__ k_cache, T* __restrict__ v_cache, PagedKV c, int32_t* __restrict__ bh_lens, int H, int G, int D,
    int Dv, int reserved_slot, Rotation rot, int norm) {
  extern __shared__ float rot_cs[];   // cos [dims / 2], sin [dims / 2]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = token_slot[t];
  const int pos = positions[t];
  const int half = rot.inv_freq ? rot.dims / 2 : 0;
  const float* cs = rot_cs;
  const float* sn = rot_cs + half;
  if (half > 0) {
    fill_rotation(rot_cs, rot_cs + half, rot, pos);
    __syncthreads();
  }
  const T* row = qkv + (int64_t)t * qkv_stride;
  const int pairs = (D + 1) / 2;
  for (int r = warp; r < H + 2 * G; r += 4) {
    if (r < H + G) {
      const bool is_q = r < H;
      const T* src = row + (int64_t)r * D;  // k heads follow the q heads with the same row size
      if (!is_q && slot == reserved_slot) continue;
      // a lane takes pairs of neighbours, so that a rotated pair stays in one lane
      auto pair_at = [&](int p, float& a, float& b) {
        a = to_f<T>(src[2 * p]);
        b = 2 * p + 1 < D ? to_f<T>(src[2 * p + 1]) : 0.f;
        if (p < half) {
          const float u = a, v = b;
          a = u * cs[p] - v * sn[p];
          b = v * cs[p] + u * sn[p];
        }
      };
      float ss = 0.f;
      for (int p = lane; p < pairs; p += 32) {
        float a, b;
        pair_at(p, a, b);
        ss += a * a + b * b;
      }
      ss = warp_sum(ss);
      const float inv = norm ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;
      const float* w = norm ? (is_q ? q_w : k_w) : nullptr;
      T* dst = is_q ? q_out + ((int64_t)t * H + r) * D : k_cache + cache_row(c, slot, r - H, pos) * D;
      for (int p = lane; p < pairs; p += 32) {
        float a, b;
        pair_at(p, a, b);
        a *= inv;
        b *= inv;
        dst[2 * p] = from_f<T>(w ? a * w[2 * p] : a);
        if (2 * p + 1 < D) dst[2 * p + 1] = from_f<T>(w ? b * w[2 * p + 1] : b);
      }
    } else {
      if (slot == reserved_slot) continue;
      const int g = r - H - G;
      const T* src = row + (int64_t)(H + G) * D + (int64_t)g * Dv;
      T* dst = v_cache + cache_row(c, slot, g, pos) * Dv;
      for (int d = lane; d < Dv; d += 32) dst[d] = src[d];
      if (lane == 0 && bh_lens) atomicMax(bh_lens + slot * G + g, pos + 1);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Portions.  CTA = (64-query tile of one sequence's new tokens, query head); 256 threads as 16 x 16: thread
// (ty, tx) owns query rows 4 ty .. 4 ty + 3, score columns tx + 16 j and output columns tx + 16 c.
// ---------------------------------------------------------------------------------------------------------
constexpr int BM = 64;

template <typename T, int BN, int DVC>
__global__ void __launch_bounds__(256) bias_attn_varlen_kernel(
    const T* __restrict__ q, PagedKV c, const int32_t* __restrict__ cu_q, const int32_t* __restrict__ seq_start,
    const int32_t* __restrict__ batch_mapping, const float* __restrict__ slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale,
    T* __restrict__ out, int H, int G, int D, int Dv) {
  constexpr int NJ = BN / 16;
  const int b = blockIdx.y, h = blockIdx.z;
  const int q0 = cu_q[b], n_new = cu_q[b + 1] - q0;
  const int tile0 = blockIdx.x * BM;
  if (tile0 >= n_new) return;
  const int slot = batch_mapping[b];
  const int g = h / (H / G);
  const int start = seq_start[b];
  const int rows = min(BM, n_new - tile0);
  const int p_first = start + tile0, p_last = p_first + rows - 1;
  const int lo = first_key(p_first, chunk, db);
  const float slope = slopes ? slopes[h] : 0.f;

  extern __shared__ float smem[];
  __shared__ int64_t rix[BN];       // cache row of every key of the tile
  const int DP = D + 1;
  float* Qs = smem;                 // [BM][DP]
  float* Ks = Qs + BM * DP;         // [BN][DP]
  float* Vs = Ks + BN * DP;         // [BN][Dv]
  float* Ps = Vs + BN * Dv;         // [BM][BN + 1]
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;

  for (int i = tid; i < BM * D; i += 256) {
    const int r = i / D, d = i - r * D;
    Qs[r * DP + d] = r < rows ? to_f<T>(q[((int64_t)(q0 + tile0 + r) * H + h) * D + d]) : 0.f;
  }
  float m[4], l[4], acc[4][DVC];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // with a sink the running maximum starts at the sink's score and the running sum with its term
    m[i] = sink > 0.f ? (sink_logits ? sink_logits[h] : 0.f) : -INFINITY;
    l[i] = sink;
#pragma unroll
    for (int cc = 0; cc < DVC; ++cc) acc[i][cc] = 0.f;
  }
  const T* kc = static_cast<const T*>(c.k);
  const T* vc = static_cast<const T*>(c.v);

  for (int k0 = lo; k0 <= p_last; k0 += BN) {
    __syncthreads();  // the previous tile's Ks / Vs / Ps are no longer read
    const int nk = min(BN, p_last + 1 - k0);
    if (tid < nk) rix[tid] = cache_row(c, slot, g, k0 + tid);
    __syncthreads();
    for (int i = tid; i < BN * D; i += 256) {
      const int r = i / D, d = i - r * D;
      Ks[r * DP + d] = r < nk ? to_f<T>(kc[rix[r] * D + d]) : 0.f;
    }
    for (int i = tid; i < BN * Dv; i += 256) {
      const int r = i / Dv, d = i - r * Dv;
      Vs[i] = r < nk ? to_f<T>(vc[rix[r] * c.v_stride + d]) : 0.f;
    }
    __syncthreads();
    float s[4][NJ];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < NJ; ++j) s[i][j] = 0.f;
    for (int d = 0; d < D; ++d) {
      float qv[4], kv[NJ];
#pragma unroll
      for (int i = 0; i < 4; ++i) qv[i] = Qs[(ty * 4 + i) * DP + d];
#pragma unroll
      for (int j = 0; j < NJ; ++j) kv[j] = Ks[(tx + 16 * j) * DP + d];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < NJ; ++j) s[i][j] = fmaf(qv[i], kv[j], s[i][j]);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = ty * 4 + i;
      const int pi = p_first + r;
      const int lo_i = first_key(pi, chunk, db);
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const int pj = k0 + tx + 16 * j;
        const bool ok = r < rows && pj <= pi && pj >= lo_i;
        s[i][j] = ok ? s[i][j] * scale - slope * (float)(pi - pj) + dist_bias_at(db, pi - pj, H, h) : -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      const float m_new = fmaxf(m[i], mx);
      // m_new == -inf: no key seen so far and none in this tile; everything stays zero
      const float corr = m_new == -INFINITY ? 1.f : expf(m[i] - m_new);
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        const float p = s[i][j] == -INFINITY ? 0.f : expf(s[i][j] - m_new);
        Ps[r * (BN + 1) + tx + 16 * j] = p;
        sum += p;
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      l[i] = l[i] * corr + sum;
      m[i] = m_new;
#pragma unroll
      for (int cc = 0; cc < DVC; ++cc) acc[i][cc] *= corr;
    }
    __syncthreads();
    for (int j = 0; j < nk; ++j) {
      float pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = Ps[(ty * 4 + i) * (BN + 1) + j];
#pragma unroll
      for (int cc = 0; cc < DVC; ++cc) {
        const int col = tx + 16 * cc;
        if (col < Dv) {
          const float vv = Vs[j * Dv + col];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i][cc] = fmaf(pv[i], vv, acc[i][cc]);
        }
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = ty * 4 + i;
    if (r >= rows) continue;
    const float inv = l[i] > 0.f ? 1.0f / l[i] : 0.f;
#pragma unroll
    for (int cc = 0; cc < DVC; ++cc) {
      const int col = tx + 16 * cc;
      if (col < Dv) out[((int64_t)(q0 + tile0 + r) * H + h) * Dv + col] = from_f<T>(acc[i][cc] * inv);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------
// Portions, tensor-core path: bfloat16, D a multiple of 16, Dv a multiple of 8, both at most DMAX (64 or 128).
// CTA = (64-query tile, query head), 4 warps; warp w owns query rows 16 w .. 16 w + 15 of the tile and keeps their
// Q fragments, running maxima and sums, and output accumulators in registers.  Keys and values come in tiles of 64
// rows through shared memory (16-byte copies out of the paged cache).  S = Q K^T and O += P V are
// mma.sync m16n8k16 with fp32 accumulators; bias, masks and the softmax run in fp32 on the S fragments, P is rounded
// to bfloat16 for the second product.
// ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_row);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// 16 bytes global -> shared without passing through registers; bytes == 0 writes zeros and reads nothing
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, int bytes) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(addr), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int DMAX>
__global__ void __launch_bounds__(128) bias_attn_varlen_mma_kernel(
    const __nv_bfloat16* __restrict__ q, PagedKV c, const int32_t* __restrict__ cu_q,
    const int32_t* __restrict__ seq_start, const int32_t* __restrict__ batch_mapping,
    const float* __restrict__ slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale, __nv_bfloat16* __restrict__ out, int H, int G,
    int D, int Dv) {
  constexpr int BN = 64, LD = DMAX + 8, KS = DMAX / 16, NV = DMAX / 8;
  constexpr float kL2e = 1.4426950408889634f;   // scores in log2 units: one ex2.approx per exponential
  typedef __nv_bfloat16 Tile[BN][LD];
  extern __shared__ __align__(16) unsigned char dyn_smem[];
  Tile* Ks = reinterpret_cast<Tile*>(dyn_smem);   // two stages of keys, then two stages of values
  Tile* Vs = Ks + 2;
  const int b = blockIdx.y, h = blockIdx.z;
  const int q0 = cu_q[b], n_new = cu_q[b + 1] - q0;
  // the latest (heaviest) query tiles first
  const int tile0 = ((int)gridDim.x - 1 - (int)blockIdx.x) * BM;
  if (tile0 >= n_new) return;
  const int slot = batch_mapping[b];
  const int g = h / (H / G);
  const int rows = min(BM, n_new - tile0);
  const int p_first = seq_start[b] + tile0, p_last = p_first + rows - 1;
  const int lo = first_key(p_first, chunk, db);
  const float slope2 = slopes ? slopes[h] * kL2e : 0.f;
  const float scale2 = scale * kL2e;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, quad = lane >> 2, tq = lane & 3;
  const int r_lo = warp * 16 + quad, r_hi = r_lo + 8;           // this lane's two query rows of the tile
  const __nv_bfloat16* kc = static_cast<const __nv_bfloat16*>(c.k);
  const __nv_bfloat16* vc = static_cast<const __nv_bfloat16*>(c.v);
  const int kvec = D / 8, vvec = Dv / 8;

  auto issue_tile = [&](int stage, int k0) {
    const int nk = min(BN, p_last + 1 - k0);
    for (int i = tid; i < BN * kvec; i += 128) {
      const int r = i / kvec, cv = i - r * kvec;
      const bool in = r < nk;
      cp_async16(&Ks[stage][r][cv * 8], in ? kc + cache_row(c, slot, g, k0 + r) * D + cv * 8 : kc, in ? 16 : 0);
    }
    for (int i = tid; i < BN * (DMAX / 8); i += 128) {   // every column of the tile: unused ones must not hold NaN
      const int r = i / (DMAX / 8), cv = i - r * (DMAX / 8);
      const bool in = r < nk && cv < vvec;
      cp_async16(&Vs[stage][r][cv * 8], in ? vc + cache_row(c, slot, g, k0 + r) * c.v_stride + cv * 8 : vc, in ? 16 : 0);
    }
    cp_async_commit();
  };
  issue_tile(0, lo);

  uint32_t qa[KS][4];
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const int col = ks * 16 + tq * 2;
    const __nv_bfloat16* row_lo = q + ((int64_t)(q0 + tile0 + r_lo) * H + h) * D;
    const __nv_bfloat16* row_hi = q + ((int64_t)(q0 + tile0 + r_hi) * H + h) * D;
    const bool in = ks * 16 < D;
    qa[ks][0] = (in && r_lo < rows) ? *reinterpret_cast<const uint32_t*>(row_lo + col) : 0u;
    qa[ks][1] = (in && r_hi < rows) ? *reinterpret_cast<const uint32_t*>(row_hi + col) : 0u;
    qa[ks][2] = (in && r_lo < rows) ? *reinterpret_cast<const uint32_t*>(row_lo + col + 8) : 0u;
    qa[ks][3] = (in && r_hi < rows) ? *reinterpret_cast<const uint32_t*>(row_hi + col + 8) : 0u;
  }
  float m[2], l[2], o[NV][4];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    m[i] = sink > 0.f ? (sink_logits ? sink_logits[h] * kL2e : 0.f) : -INFINITY;   // with a sink: its score and its term
    l[i] = sink;
  }
#pragma unroll
  for (int nb = 0; nb < NV; ++nb)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nb][e] = 0.f;
  const int pi_lo = p_first + r_lo, pi_hi = p_first + r_hi;
  const int lo_lo = first_key(pi_lo, chunk, db), lo_hi = first_key(pi_hi, chunk, db);
  // a tile needs no masks for this warp when all its keys are at or before the warp's first row and inside the
  // chunk of the warp's last row (rows beyond `rows` are never written, their values do not matter)
  const int warp_first = p_first + warp * 16;
  const int warp_lo = first_key(warp_first + 15, chunk, db);

  int stage = 0;
  for (int k0 = lo; k0 <= p_last; k0 += BN, stage ^= 1) {
    const int nk = min(BN, p_last + 1 - k0);
    if (k0 + BN <= p_last) {
      issue_tile(stage ^ 1, k0 + BN);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();   // every thread's copies of this stage have landed
    float s[BN / 8][4];
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[nb][e] = 0.f;
    // k-steps outside, key blocks inside: eight independent accumulator chains are in flight per k-step
#pragma unroll
    for (int ks = 0; ks < KS; ks += 2) {
      if (ks * 16 < D) {
#pragma unroll
        for (int nb = 0; nb < BN / 8; ++nb) {
          uint32_t kb[4];
          ldmatrix_x4(kb, &Ks[stage][nb * 8 + (lane & 7)][ks * 16 + (lane >> 3) * 8]);
          mma16816<true>(s[nb], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], kb[0], kb[1]);
          if ((ks + 1) * 16 < D)
            mma16816<true>(s[nb], qa[ks + 1][0], qa[ks + 1][1], qa[ks + 1][2], qa[ks + 1][3], kb[2], kb[3]);
        }
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
    if (k0 + BN - 1 <= warp_first && k0 >= warp_lo) {
#pragma unroll
      for (int nb = 0; nb < BN / 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int pj = k0 + nb * 8 + tq * 2 + (e & 1);
          const int dist = ((e & 2) ? pi_hi : pi_lo) - pj;
          s[nb][e] = s[nb][e] * scale2 - slope2 * (float)dist + dist_bias_at(db, dist, H, h) * kL2e;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
        }
    } else {
#pragma unroll
      for (int nb = 0; nb < BN / 8; ++nb)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int pj = k0 + nb * 8 + tq * 2 + (e & 1);
          const int pi = (e & 2) ? pi_hi : pi_lo;
          const int lo_i = (e & 2) ? lo_hi : lo_lo;
          const bool ok = ((e & 2) ? r_hi : r_lo) < rows && pj <= pi && pj >= lo_i;
          s[nb][e] = ok ? s[nb][e] * scale2 - slope2 * (float)(pi - pj) + dist_bias_at(db, pi - pj, H, h) * kL2e
                        : -INFINITY;
          mx[e >> 1] = fmaxf(mx[e >> 1], s[nb][e]);
        }
    }
    float corr[2], mref[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float m_new = fmaxf(m[i], mx[i]);
      // no key seen so far and none in this tile: nothing to rescale, and a finite stand-in keeps ex2(-inf - m) = 0
      corr[i] = m_new == -INFINITY ? 1.f : ex2(m[i] - m_new);
      mref[i] = m_new == -INFINITY ? 0.f : m_new;
      m[i] = m_new;
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int nb = 0; nb < BN / 8; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float p = ex2(s[nb][e] - mref[e >> 1]);   // masked scores are -inf: ex2 gives 0
        s[nb][e] = p;
        sum[e >> 1] += p;
      }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
      l[i] = l[i] * corr[i] + sum[i];
    }
#pragma unroll
    for (int nb = 0; nb < NV; ++nb) {
      o[nb][0] *= corr[0];
      o[nb][1] *= corr[0];
      o[nb][2] *= corr[1];
      o[nb][3] *= corr[1];
    }
#pragma unroll
    for (int kb = 0; kb < BN / 16; ++kb) {
      if (kb * 16 < nk) {
        const uint32_t a0 = pack2<true>(s[2 * kb][0], s[2 * kb][1]), a1 = pack2<true>(s[2 * kb][2], s[2 * kb][3]);
        const uint32_t a2 = pack2<true>(s[2 * kb + 1][0], s[2 * kb + 1][1]);
        const uint32_t a3 = pack2<true>(s[2 * kb + 1][2], s[2 * kb + 1][3]);
#pragma unroll
        for (int nb = 0; nb < NV; nb += 2) {
          if (nb * 8 < Dv) {
            uint32_t vb[4];
            ldmatrix_x4_trans(vb, &Vs[stage][kb * 16 + (lane & 15)][nb * 8 + (lane >> 4) * 8]);
            mma16816<true>(o[nb], a0, a1, a2, a3, vb[0], vb[1]);
            mma16816<true>(o[nb + 1], a0, a1, a2, a3, vb[2], vb[3]);
          }
        }
      }
    }
    __syncthreads();   // the stage is free for the copy the next pass issues
  }
  const float inv[2] = {l[0] > 0.f ? 1.0f / l[0] : 0.f, l[1] > 0.f ? 1.0f / l[1] : 0.f};
#pragma unroll
  for (int nb = 0; nb < NV; ++nb) {
    const int col = nb * 8 + tq * 2;
    if (col < Dv) {
      if (r_lo < rows)
        *reinterpret_cast<uint32_t*>(out + ((int64_t)(q0 + tile0 + r_lo) * H + h) * Dv + col) =
            pack2<true>(o[nb][0] * inv[0], o[nb][1] * inv[0]);
      if (r_hi < rows)
        *reinterpret_cast<uint32_t*>(out + ((int64_t)(q0 + tile0 + r_hi) * H + h) * Dv + col) =
            pack2<true>(o[nb][2] * inv[1], o[nb][3] * inv[1]);
    }
  }
}

template <int DMAX>
int launch_varlen_mma(const void* q, const PagedKV& c, const int32_t* cu_q, const int32_t* seq_start, const int32_t* bm,
                      const float* slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale, void* out, int B, int max_new, int H,
                      int G, int D, int Dv, cudaStream_t st) {
  static std::atomic<uint64_t> mask{0};
  const int smem = 4 * 64 * (DMAX + 8) * 2;
  auto kern = bias_attn_varlen_mma_kernel<DMAX>;
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem(reinterpret_cast<const void*>(kern), smem, mask));
  dim3 grid(cdiv(max_new, BM), B, H);
  kern<<<grid, 128, smem, st>>>(static_cast<const __nv_bfloat16*>(q), c, cu_q, seq_start, bm, slopes, chunk, db, sink, sink_logits,
                                scale, static_cast<__nv_bfloat16*>(out), H, G, D, Dv);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Decode.  CTA = (sequence, query head), 4 warps; a warp takes 32 keys at a time, one key per lane for the
// score, one output column per lane (and every 32nd after it) for the value sum; the warps' partial softmax
// states are merged through shared memory.
// ---------------------------------------------------------------------------------------------------------
constexpr int kDecWarps = 4;
constexpr int kDecCols = 16;  // output columns per lane: Dv <= 512

template <typename T>
__global__ void __launch_bounds__(kDecWarps * 32) bias_attn_decode_kernel(
    const T* __restrict__ q, PagedKV c, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ batch_mapping, const float* __restrict__ slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale,
    T* __restrict__ out, int H, int G, int D, int Dv, int reserved_slot) {
  extern __shared__ float smem[];
  float* qs = smem;                         // [D]
  float* part = qs + D;                     // [kDecWarps][2 + Dv]
  const int b = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = batch_mapping[b];
  T* o = out + ((int64_t)b * H + h) * Dv;
  if (slot == reserved_slot) {
    for (int d = threadIdx.x; d < Dv; d += blockDim.x) o[d] = from_f<T>(0.f);
    return;
  }
  const int g = h / (H / G);
  const int pi = positions[b];
  const int lo = first_key(pi, chunk, db);
  const float slope = slopes ? slopes[h] : 0.f;
  for (int d = threadIdx.x; d < D; d += blockDim.x) qs[d] = to_f<T>(q[((int64_t)b * H + h) * D + d]);
  __syncthreads();
  const T* kc = static_cast<const T*>(c.k);
  const T* vc = static_cast<const T*>(c.v);
  float m = -INFINITY, l = 0.f, acc[kDecCols];
#pragma unroll
  for (int cc = 0; cc < kDecCols; ++cc) acc[cc] = 0.f;
  for (int k0 = lo + warp * 32; k0 <= pi; k0 += kDecWarps * 32) {
    const int pj = k0 + lane;
    const bool ok = pj <= pi;
    const int64_t row = ok ? cache_row(c, slot, g, pj) : 0;
    float s = -INFINITY;
    if (ok) {
      const T* kr = kc + row * D;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot = fmaf(qs[d], to_f<T>(kr[d]), dot);
      s = dot * scale - slope * (float)(pi - pj) + dist_bias_at(db, pi - pj, H, h);
    }
    const float m_new = fmaxf(m, warp_max(s));  // lane 0 of the batch is always a live key
    const float corr = expf(m - m_new);
    const float p = ok ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int cc = 0; cc < kDecCols; ++cc) acc[cc] *= corr;
    const int nk = min(32, pi + 1 - k0);
    for (int j = 0; j < nk; ++j) {
      const float pj_w = __shfl_sync(0xffffffffu, p, j);
      const int64_t rj = __shfl_sync(0xffffffffu, row, j);
      const T* vr = vc + rj * c.v_stride;
#pragma unroll
      for (int cc = 0; cc < kDecCols; ++cc) {
        const int col = lane + 32 * cc;
        if (col < Dv) acc[cc] = fmaf(pj_w, to_f<T>(vr[col]), acc[cc]);
      }
    }
  }
  float* mine = part + warp * (2 + Dv);
  if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
  for (int cc = 0; cc < kDecCols; ++cc) {
    const int col = lane + 32 * cc;
    if (col < Dv) mine[2 + col] = acc[cc];
  }
  __syncthreads();
  const float sink_m = sink_logits ? sink_logits[h] : 0.f;   // the sink's score
  float mm = sink > 0.f ? sink_m : -INFINITY;
  for (int w = 0; w < kDecWarps; ++w) mm = fmaxf(mm, part[w * (2 + Dv)]);
  float ll = sink > 0.f ? sink * expf(sink_m - mm) : 0.f;
  float f[kDecWarps];
  for (int w = 0; w < kDecWarps; ++w) {
    const float mw = part[w * (2 + Dv)];
    f[w] = mw == -INFINITY ? 0.f : expf(mw - mm);
    ll += part[w * (2 + Dv) + 1] * f[w];
  }
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
  for (int d = threadIdx.x; d < Dv; d += blockDim.x) {
    float a = 0.f;
    for (int w = 0; w < kDecWarps; ++w) a += part[w * (2 + Dv) + 2 + d] * f[w];
    o[d] = from_f<T>(a * inv);
  }
}


// ---------------------------------------------------------------------------------------------------------
// Decode, vector path (D and Dv multiples of 8, at most 256).  CTA = (key split, kv head x tile of up to four of
// its query heads, sequence); 128 threads = 16 groups of 8 lanes.  A group takes every 16th key of the split: its
// lanes read the key row and the value row in 16-byte pieces (lane `sub` owns elements 8 (sub + 8 i) ... + 7), the
// dot products of the tile's heads are finished by three shuffles inside the group, and each group carries its own
// running softmax state.  The states are merged by shuffles inside a warp, through shared memory across warps, and
// - with more than one split - by bias_attn_decode_merge_kernel from a workspace of (max, sum, values) records.
// ---------------------------------------------------------------------------------------------------------
// largest CH (64-column chunks of the head size) whose query slice the decode kernel keeps in registers
#ifndef CVLLM_DEC_QREG_CH
#define CVLLM_DEC_QREG_CH 2
#endif
constexpr int kDecTile = 4;   // query heads per CTA
// scores are kept in log2 units (log2(e) folded into the query scale and the slopes), so every exponential of the
// split and merge kernels is one ex2.approx
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kDecSlack = 8.f;   // how far a logit may pass the running reference point before it moves

template <typename T>
__device__ __forceinline__ void load8(const T* p, float* v);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float* v) {
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <>
__device__ __forceinline__ void load8<float>(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float* v);
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float* v) {
  *reinterpret_cast<uint4*>(p) = make_uint4(pack2<true>(v[0], v[1]), pack2<true>(v[2], v[3]), pack2<true>(v[4], v[5]),
                                            pack2<true>(v[6], v[7]));
}
template <>
__device__ __forceinline__ void store8<float>(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
}

// q / k norm + store with 16-byte accesses: D and Dv multiples of 8 and at most 256, rows 16-byte aligned.
// LPR lanes (a power of two, 8 elements each) share a head row, so a warp takes 32 / LPR rows at once and a CTA
// 4 * 32 / LPR; grid = (tokens, row groups): a decode step's few tokens still spread over many CTAs.  A lane keeps its
// piece of the row in registers between the sum of squares and the scaled write.
template <typename T>
__global__ void __launch_bounds__(128) qknorm_store_vec_kernel(
    const T* __restrict__ qkv, int64_t qkv_stride, const float* __restrict__ q_w, const float* __restrict__ k_w,
    float eps, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_slot, T* __restrict__ q_out,
    T* __restrict__ k_cache, T* __restrict__ v_cache, PagedKV c, int32_t* __restrict__ bh_lens, int H, int G, int D,
    int Dv, int reserved_slot, int lpr, Rotation rot, int norm) {
  extern __shared__ float rot_cs[];   // cos [dims / 2], sin [dims / 2]
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = token_slot[t];
  const int pos = positions[t];
  const int half = rot.inv_freq ? rot.dims / 2 : 0;
  if (half > 0) {
    fill_rotation(rot_cs, rot_cs + half, rot, pos);
    __syncthreads();
  }
  const T* row = qkv + (int64_t)t * qkv_stride;
  const int rows_per_warp = 32 / lpr;
  const int r = (blockIdx.y * 4 + warp) * rows_per_warp + lane / lpr;
  const int cb = (lane % lpr) * 8;
  const bool is_q = r < H, is_k = r >= H && r < H + G, is_v = r >= H + G && r < H + 2 * G;
  const bool stores = slot != reserved_slot;
  float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if ((is_q || (is_k && stores)) && cb < D) load8<T>(row + (int64_t)r * D + cb, x);
  if (half > 0 && (is_q || is_k)) {   // the lane's four pairs of neighbours
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
      const int p = (cb + e) >> 1;
      if (p < half) {
        const float u = x[e], v = x[e + 1];
        x[e] = u * rot_cs[p] - v * rot_cs[half + p];
        x[e + 1] = v * rot_cs[p] + u * rot_cs[half + p];
      }
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
  for (int o = lpr >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);   // every lane takes part
  if ((is_q || (is_k && stores)) && cb < D) {
    const float inv = norm ? 1.0f / sqrtf(ss / (float)D + eps) : 1.0f;
    const float* w = norm ? (is_q ? q_w : k_w) : nullptr;
#pragma unroll
    for (int e = 0; e < 8; ++e) x[e] = w ? x[e] * inv * w[cb + e] : x[e] * inv;
    T* dst = is_q ? q_out + ((int64_t)t * H + r) * D : k_cache + cache_row(c, slot, r - H, pos) * D;
    store8<T>(dst + cb, x);
  }
  if (is_v && stores) {
    const int g = r - H - G;
    if (cb < Dv) {
      float v[8];
      load8<T>(row + (int64_t)(H + G) * D + (int64_t)g * Dv + cb, v);
      store8<T>(v_cache + cache_row(c, slot, g, pos) * Dv + cb, v);
    }
    if (cb == 0 && bh_lens) atomicMax(bh_lens + slot * G + g, pos + 1);
  }
}

template <typename T, int CH>
__global__ void __launch_bounds__(128) bias_attn_decode_split_kernel(
    const T* __restrict__ q, PagedKV c, const int32_t* __restrict__ positions,
    const int32_t* __restrict__ batch_mapping, const float* __restrict__ slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale,
    T* __restrict__ out, float* __restrict__ part, int H, int G, int D, int Dv, int splits, int reserved_slot) {
  __shared__ float qs[kDecTile][64 * CH];
  __shared__ float st[4][kDecTile][2 + 64 * CH];
  const int split = blockIdx.x, b = blockIdx.z;
  const int R = H / G, tiles = (R + kDecTile - 1) / kDecTile;
  const int g = blockIdx.y / tiles, h0 = g * R + (blockIdx.y % tiles) * kDecTile;
  const int nr = min(kDecTile, g * R + R - h0);
  const int tid = threadIdx.x, sub = tid & 7, gid = tid >> 3, warp = tid >> 5;
  const int slot = batch_mapping[b];
  const int rec = 2 + Dv;
  if (slot == reserved_slot) {
    for (int i = tid; i < nr * Dv; i += 128) {
      const int r = i / Dv, d = i - r * Dv;
      if (splits == 1) out[((int64_t)b * H + h0 + r) * Dv + d] = from_f<T>(0.f);
    }
    if (splits > 1 && tid < nr) {
      float* p = part + (((int64_t)b * H + h0 + tid) * splits + split) * rec;
      p[0] = -INFINITY;
      p[1] = 0.f;
    }
    return;
  }
  const int pi = positions[b];
  const int lo = first_key(pi, chunk, db);
  const int n = pi - lo + 1, per = (n + splits - 1) / splits;
  const int k_begin = lo + split * per, k_end = min(pi + 1, k_begin + per);
  for (int i = tid; i < kDecTile * D; i += 128) {
    const int r = i / D, d = i - r * D;
    qs[r][d] = r < nr ? to_f<T>(q[((int64_t)b * H + h0 + r) * D + d]) * (scale * kLog2e) : 0.f;
  }
  float slope[kDecTile];
#pragma unroll
  for (int r = 0; r < kDecTile; ++r) slope[r] = (slopes && r < nr) ? slopes[h0 + r] * kLog2e : 0.f;
  __syncthreads();
  const T* kc = static_cast<const T*>(c.k);
  const T* vc = static_cast<const T*>(c.v);
  float m[kDecTile], l[kDecTile], acc[kDecTile][CH * 8];
#pragma unroll
  for (int r = 0; r < kDecTile; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int e = 0; e < CH * 8; ++e) acc[r][e] = 0.f;
  }
  const unsigned gmask = 0xffu << (tid & 24);   // the group's own lanes: groups of a warp leave the loop apart
  // the lane's slice of the tile's queries stays in registers when it is small enough (D <= 128)
  constexpr bool kQInRegs = CH <= CVLLM_DEC_QREG_CH;
  float qr[kQInRegs ? kDecTile : 1][kQInRegs ? CH * 8 : 1];
  if constexpr (kQInRegs) {
#pragma unroll
    for (int r = 0; r < kDecTile; ++r)
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int cb = (sub + 8 * i) * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) qr[r][i * 8 + e] = cb < D ? qs[r][cb + e] : 0.f;
      }
  }
  // Each lane streams ITS slices of the group's key and value rows through a ring of kStages entries in shared
  // memory with cp.async: kStages keys are in flight per group whatever the register budget, and a lane only ever
  // reads what it copied itself, so the ring needs no barrier - cp.async.wait_group orders a lane's own copies.
  // Entry layout [stage][K chunks | V chunks][thread]: consecutive lanes hit consecutive 16-byte words.
  constexpr int kStages = CH <= 2 ? 4 : 2;
  constexpr int kVec = 16 / sizeof(T);          // elements per 16-byte piece
  constexpr int kPieces = 8 / kVec;             // 16-byte pieces per 8-element chunk (1 for 16 bit, 2 for 32 bit)
  extern __shared__ __align__(16) unsigned char ring_raw[];
  uint4* ring = reinterpret_cast<uint4*>(ring_raw);
  auto ring_at = [&](int stage, int which, int i, int piece) -> uint4* {
    return ring + ((((stage * 2 + which) * CH + i) * kPieces + piece) * 128 + tid);
  };
  const int n_mine = k_end > k_begin + gid ? (k_end - k_begin - gid + 15) / 16 : 0;
  auto issue = [&](int t) {
    if (t < n_mine) {
      const int64_t row = cache_row(c, slot, g, k_begin + gid + 16 * t);
      const int stage = t % kStages;
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int cb = (sub + 8 * i) * 8;
#pragma unroll
        for (int pc = 0; pc < kPieces; ++pc) {
          if (cb < D) cp_async16(ring_at(stage, 0, i, pc), kc + row * D + cb + pc * kVec, 16);
          if (cb < Dv) cp_async16(ring_at(stage, 1, i, pc), vc + row * c.v_stride + cb + pc * kVec, 16);
        }
      }
    }
    cp_async_commit();   // also when empty: the group count per pass stays the same
  };
  auto read8 = [&](int stage, int which, int i, float* v) {
    if constexpr (sizeof(T) == 2) {
      const uint4 u = *ring_at(stage, which, i, 0);
      const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        v[2 * k] = __uint_as_float(w[k] << 16);
        v[2 * k + 1] = __uint_as_float(w[k] & 0xffff0000u);
      }
    } else {
      const uint4 a = *ring_at(stage, which, i, 0), b2 = *ring_at(stage, which, i, kPieces - 1);
      v[0] = __uint_as_float(a.x); v[1] = __uint_as_float(a.y); v[2] = __uint_as_float(a.z); v[3] = __uint_as_float(a.w);
      v[4] = __uint_as_float(b2.x); v[5] = __uint_as_float(b2.y); v[6] = __uint_as_float(b2.z); v[7] = __uint_as_float(b2.w);
    }
  };
#pragma unroll
  for (int t = 0; t < kStages - 1; ++t) issue(t);
  for (int t = 0; t < n_mine; ++t) {
    issue(t + kStages - 1);          // refills the entry the previous pass has finished reading
    cp_async_wait<kStages - 1>();    // everything but the newest kStages - 1 groups has landed: key t is here
    const int stage = t % kStages;
    const int j = k_begin + gid + 16 * t;
    float s[kDecTile];
#pragma unroll
    for (int r = 0; r < kDecTile; ++r) s[r] = 0.f;
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int cb = (sub + 8 * i) * 8;
      if (cb < D) {
        float kv[8];
        read8(stage, 0, i, kv);
#pragma unroll
        for (int r = 0; r < kDecTile; ++r)
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            float qv;
            if constexpr (kQInRegs) qv = qr[r][i * 8 + e];
            else qv = qs[r][cb + e];
            s[r] = fmaf(qv, kv[e], s[r]);
          }
      }
    }
    const float dist = (float)(pi - j);
    float p[kDecTile];
#pragma unroll
    for (int r = 0; r < kDecTile; ++r) {
      float v = s[r];
      v += __shfl_xor_sync(gmask, v, 4);
      v += __shfl_xor_sync(gmask, v, 2);
      v += __shfl_xor_sync(gmask, v, 1);
      v -= slope[r] * dist;
      if (db.table != nullptr && r < nr) v += dist_bias_at(db, pi - j, H, h0 + r) * kLog2e;
      // The reference point m moves only when a logit passes it by more than kDecSlack (log2 units): weights stay
      // below 2^kDecSlack, far inside fp32, and the result is the same sum.  With a distance bias the logits of
      // later keys keep rising, so an exact running maximum would rescale the accumulators at almost every key.
      if (v > m[r] + kDecSlack) {   // the same for the 8 lanes of the group
        const float corr = ex2(m[r] - v);
        l[r] *= corr;
#pragma unroll
        for (int e = 0; e < CH * 8; ++e) acc[r][e] *= corr;
        m[r] = v;
      }
      p[r] = ex2(v - m[r]);
      l[r] += p[r];
    }
#pragma unroll
    for (int i = 0; i < CH; ++i) {
      const int cb = (sub + 8 * i) * 8;
      if (cb < Dv) {
        float vv[8];
        read8(stage, 1, i, vv);
#pragma unroll
        for (int r = 0; r < kDecTile; ++r)
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[r][i * 8 + e] = fmaf(p[r], vv[e], acc[r][i * 8 + e]);
      }
    }
  }
  cp_async_wait<0>();
  // the four groups of a warp (lanes differing in bits 3 and 4)
#pragma unroll
  for (int o = 8; o <= 16; o <<= 1) {
#pragma unroll
    for (int r = 0; r < kDecTile; ++r) {
      const float mo = __shfl_xor_sync(0xffffffffu, m[r], o);
      const float lo_ = __shfl_xor_sync(0xffffffffu, l[r], o);
      const float mn = fmaxf(m[r], mo);
      const float fa = m[r] == -INFINITY ? 0.f : ex2(m[r] - mn);
      const float fb = mo == -INFINITY ? 0.f : ex2(mo - mn);
      l[r] = l[r] * fa + lo_ * fb;
#pragma unroll
      for (int e = 0; e < CH * 8; ++e) {
        const float ao = __shfl_xor_sync(0xffffffffu, acc[r][e], o);
        acc[r][e] = acc[r][e] * fa + ao * fb;
      }
      m[r] = mn;
    }
  }
  if ((tid & 31) < 8) {
#pragma unroll
    for (int r = 0; r < kDecTile; ++r) {
      if (sub == 0) { st[warp][r][0] = m[r]; st[warp][r][1] = l[r]; }
#pragma unroll
      for (int i = 0; i < CH; ++i) {
        const int cb = (sub + 8 * i) * 8;
        if (cb < Dv)
#pragma unroll
          for (int e = 0; e < 8; ++e) st[warp][r][2 + cb + e] = acc[r][i * 8 + e];
      }
    }
  }
  __syncthreads();
  for (int i = tid; i < nr * Dv; i += 128) {
    const int r = i / Dv, d = i - r * Dv;
    const float sink_m = sink_logits ? sink_logits[h0 + r] * 1.4426950408889634f : 0.f;   // the sink's score, log2 units
    float mm = (splits == 1 && sink > 0.f) ? sink_m : -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mm = fmaxf(mm, st[w][r][0]);
    float ll = (splits == 1 && sink > 0.f) ? sink * ex2(sink_m - mm) : 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = st[w][r][0];
      if (mw == -INFINITY) continue;
      const float f = ex2(mw - mm);
      ll += st[w][r][1] * f;
      a += st[w][r][2 + d] * f;
    }
    if (splits == 1) {
      out[((int64_t)b * H + h0 + r) * Dv + d] = from_f<T>(ll > 0.f ? a / ll : 0.f);
    } else {
      float* pr = part + (((int64_t)b * H + h0 + r) * splits + split) * rec;
      if (d == 0) { pr[0] = mm; pr[1] = ll; }
      pr[2 + d] = a;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) bias_attn_decode_merge_kernel(const float* __restrict__ part, float sink,
                                                                     const float* __restrict__ sink_logits, int H,
                                                                     T* __restrict__ out, int Dv, int splits) {
  const int64_t bh = blockIdx.x;
  const int rec = 2 + Dv;
  const float* p = part + bh * splits * rec;
  const float sink_m = sink_logits ? sink_logits[bh % H] * 1.4426950408889634f : 0.f;   // log2 units, as the parts
  float mm = sink > 0.f ? sink_m : -INFINITY;
  for (int s = 0; s < splits; ++s) mm = fmaxf(mm, p[s * rec]);
  float ll = sink > 0.f ? sink * ex2(sink_m - mm) : 0.f;
  for (int s = 0; s < splits; ++s)
    if (p[s * rec] != -INFINITY) ll += p[s * rec + 1] * ex2(p[s * rec] - mm);
  const float inv = ll > 0.f ? 1.0f / ll : 0.f;
  for (int d = threadIdx.x; d < Dv; d += 128) {
    float a = 0.f;
    for (int s = 0; s < splits; ++s)
      if (p[s * rec] != -INFINITY) a += p[s * rec + 2 + d] * ex2(p[s * rec] - mm);
    out[bh * Dv + d] = from_f<T>(a * inv);
  }
}

template <typename T, int CH>
int launch_decode_split_ch(const void* q, const PagedKV& c, const int32_t* positions, const int32_t* bm,
                           const float* slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale, void* out, float* part, dim3 grid,
                           int H, int G, int D, int Dv, int splits, int reserved_slot, cudaStream_t st) {
  // the ring: stages x (K | V) x CH chunks x 16-byte pieces per chunk x 128 threads x 16 bytes
  const size_t ring = (size_t)(CH <= 2 ? 4 : 2) * 2 * CH * (8 / (16 / sizeof(T))) * 128 * 16;
  static std::atomic<uint64_t> mask{0};
  auto kern = bias_attn_decode_split_kernel<T, CH>;
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem(reinterpret_cast<const void*>(kern), (int)ring, mask));
  kern<<<grid, 128, ring, st>>>(static_cast<const T*>(q), c, positions, bm, slopes, chunk, db, sink, sink_logits, scale,
                                static_cast<T*>(out), part, H, G, D, Dv, splits, reserved_slot);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

template <typename T>
int launch_decode_split(const void* q, const PagedKV& c, const int32_t* positions, const int32_t* bm,
                        const float* slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale, void* out, float* part, int B, int H,
                        int G, int D, int Dv, int splits, int reserved_slot, cudaStream_t st) {
  const int R = H / G, tiles = cdiv(R, kDecTile);
  dim3 grid(splits, G * tiles, B);
  const int ch = cdiv(D > Dv ? D : Dv, 64);
  int rc;
#define CVLLM_GO(CH) \
  rc = launch_decode_split_ch<T, CH>(q, c, positions, bm, slopes, chunk, db, sink, sink_logits, scale, out, part, grid, H, G, D, Dv, \
                                     splits, reserved_slot, st)
  if (ch == 1) CVLLM_GO(1);
  else if (ch == 2) CVLLM_GO(2);
  else if (ch == 3) CVLLM_GO(3);
  else CVLLM_GO(4);
#undef CVLLM_GO
  if (rc != CVLLM_OK) return rc;
  if (splits > 1) {
    bias_attn_decode_merge_kernel<T><<<B * H, 128, 0, st>>>(part, sink, sink_logits, H, static_cast<T*>(out), Dv, splits);
    CVLLM_CHECK_LAUNCH();
  }
  return CVLLM_OK;
}

size_t varlen_smem(int BN, int D, int Dv) {
  return sizeof(float) * ((size_t)BM * (D + 1) + (size_t)BN * (D + 1) + (size_t)BN * Dv + (size_t)BM * (BN + 1));
}

template <typename T, int BN, int DVC>
int launch_varlen(const void* q, const PagedKV& c, const int32_t* cu_q, const int32_t* seq_start,
                  const int32_t* batch_mapping, const float* slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale, void* out,
                  int B, int max_new, int H, int G, int D, int Dv, cudaStream_t st) {
  static std::atomic<uint64_t> mask{0};
  const size_t smem = varlen_smem(BN, D, Dv);
  auto kern = bias_attn_varlen_kernel<T, BN, DVC>;
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem(reinterpret_cast<const void*>(kern), 226 * 1024, mask));
  dim3 grid(cdiv(max_new, BM), B, H);
  kern<<<grid, 256, smem, st>>>(static_cast<const T*>(q), c, cu_q, seq_start, batch_mapping, slopes, chunk, db, sink, sink_logits,
                                scale, static_cast<T*>(out), H, G, D, Dv);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

template <typename T, int BN>
int dispatch_dvc(int dvc, const void* q, const PagedKV& c, const int32_t* cu_q, const int32_t* seq_start,
                 const int32_t* bm, const float* slopes, int chunk, DistBias db, float sink, const float* __restrict__ sink_logits, float scale, void* out, int B,
                 int max_new, int H, int G, int D, int Dv, cudaStream_t st) {
#define CVLLM_GO(N) \
  return launch_varlen<T, BN, N>(q, c, cu_q, seq_start, bm, slopes, chunk, db, sink, sink_logits, scale, out, B, max_new, H, G, D, Dv, st)
  if (dvc <= 4) CVLLM_GO(4);
  if (dvc <= 6) CVLLM_GO(6);
  if (dvc <= 8) CVLLM_GO(8);
  if (dvc <= 16) CVLLM_GO(16);
  CVLLM_GO(32);
#undef CVLLM_GO
}

}  // namespace
}  // namespace cvllm

using namespace cvllm;

// prefill_attn_bias.cu: the tcgen05 / TMEM / TMA pipeline for 16-bit storage, D = Dv = 128, pages of a multiple of 128
// rows and an even number of query heads per KV head
int cvllm_launch_prefill_bias(const void* q, const void* k_cache, const void* v_cache, int64_t cache_rows, void* out,
                              const int32_t* seq_start, const float* slopes, const int32_t* page_table,
                              const int32_t* batch_mapping, const int32_t* cu_seqlens_q, int B, int N, int HQ, int HKV,
                              int PS, int NLP, int max_seqlen_q, float scale, int chunk, int sink, const float* sink_logits,
                              cudaStream_t st);

static int check_dtype(int dtype) { return dtype == CVLLM_BF16 || dtype == CVLLM_F32; }

static int rope_qknorm_store_impl(const double* inv_freq, int rot_dims, int norm, const void* qkv, int64_t qkv_stride, const float* q_weight, const float* k_weight,
                                  float eps, const int32_t* positions, const int32_t* token_slot, void* q_out,
                                  void* k_cache, void* v_cache, const int32_t* page_table, int64_t table_stride_slot,
                                  int64_t table_stride_head, int page_size, int32_t* bh_lens, int T, int H, int G,
                                  int D, int Dv, int reserved_slot, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(T >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0 && page_size > 0);
  CVLLM_CHECK_ARG(inv_freq == nullptr || (rot_dims >= 0 && rot_dims % 2 == 0 && rot_dims <= D));
  const Rotation rot{rot_dims > 0 ? inv_freq : nullptr, rot_dims};
  const size_t rsmem = rot.inv_freq ? sizeof(float) * (size_t)rot_dims : 0;
  CVLLM_CHECK_SUPPORTED(rsmem <= 32 * 1024);
  if (T == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(qkv && positions && token_slot && q_out && k_cache && v_cache && page_table && check_dtype(dtype));
  auto st = static_cast<cudaStream_t>(stream);
  const PagedKV c = make_paged(k_cache, v_cache, page_table, table_stride_slot, table_stride_head, page_size, Dv);
  const int64_t align = dtype == CVLLM_BF16 ? 8 : 4;
  if (D % 8 == 0 && Dv % 8 == 0 && D <= 256 && Dv <= 256 && qkv_stride % align == 0 && aligned16(qkv) &&
      aligned16(q_out) && aligned16(k_cache) && aligned16(v_cache)) {
    int lpr = 1;   // lanes per row: the next power of two that covers the longer of the two row sizes
    while (lpr * 8 < (D > Dv ? D : Dv)) lpr <<= 1;
    const int rows_per_cta = 4 * (32 / lpr);
    CVLLM_CHECK_SUPPORTED(T <= 2147483647 && cdiv(H + 2 * G, rows_per_cta) <= 65535);
    const dim3 grid(T, cdiv(H + 2 * G, rows_per_cta));
    if (dtype == CVLLM_BF16)
      qknorm_store_vec_kernel<__nv_bfloat16><<<grid, 128, rsmem, st>>>(
          static_cast<const __nv_bfloat16*>(qkv), qkv_stride, q_weight, k_weight, eps, positions, token_slot,
          static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache),
          static_cast<__nv_bfloat16*>(v_cache), c, bh_lens, H, G, D, Dv, reserved_slot, lpr, rot, norm);
    else
      qknorm_store_vec_kernel<float><<<grid, 128, rsmem, st>>>(static_cast<const float*>(qkv), qkv_stride, q_weight,
                                                           k_weight, eps, positions, token_slot,
                                                           static_cast<float*>(q_out), static_cast<float*>(k_cache),
                                                           static_cast<float*>(v_cache), c, bh_lens, H, G, D, Dv,
                                                           reserved_slot, lpr, rot, norm);
    CVLLM_CHECK_LAUNCH();
    return CVLLM_OK;
  }
  if (dtype == CVLLM_BF16)
    qknorm_store_kernel<__nv_bfloat16><<<T, 128, rsmem, st>>>(
        static_cast<const __nv_bfloat16*>(qkv), qkv_stride, q_weight, k_weight, eps, positions, token_slot,
        static_cast<__nv_bfloat16*>(q_out), static_cast<__nv_bfloat16*>(k_cache), static_cast<__nv_bfloat16*>(v_cache),
        c, bh_lens, H, G, D, Dv, reserved_slot, rot, norm);
  else
    qknorm_store_kernel<float><<<T, 128, rsmem, st>>>(static_cast<const float*>(qkv), qkv_stride, q_weight, k_weight, eps,
                                                  positions, token_slot, static_cast<float*>(q_out),
                                                  static_cast<float*>(k_cache), static_cast<float*>(v_cache), c,
                                                  bh_lens, H, G, D, Dv, reserved_slot, rot, norm);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}


extern "C" int cvllm_qknorm_store(const void* qkv, int64_t qkv_stride, const float* q_weight, const float* k_weight,
                                  float eps, const int32_t* positions, const int32_t* token_slot, void* q_out,
                                  void* k_cache, void* v_cache, const int32_t* page_table, int64_t table_stride_slot,
                                  int64_t table_stride_head, int page_size, int32_t* bh_lens, int T, int H, int G,
                                  int D, int Dv, int reserved_slot, int dtype, cvllm_stream_t stream) {
  return rope_qknorm_store_impl(nullptr, 0, 1, qkv, qkv_stride, q_weight, k_weight, eps, positions, token_slot, q_out,
                                k_cache, v_cache, page_table, table_stride_slot, table_stride_head, page_size, bh_lens,
                                T, H, G, D, Dv, reserved_slot, dtype, stream);
}

extern "C" int cvllm_rope_qknorm_store(const void* qkv, int64_t qkv_stride, const double* inv_freq, int rot_dims,
                                       int norm, const float* q_weight, const float* k_weight, float eps,
                                       const int32_t* positions, const int32_t* token_slot, void* q_out, void* k_cache,
                                       void* v_cache, const int32_t* page_table, int64_t table_stride_slot,
                                       int64_t table_stride_head, int page_size, int32_t* bh_lens, int T, int H, int G,
                                       int D, int Dv, int reserved_slot, int dtype, cvllm_stream_t stream) {
  return rope_qknorm_store_impl(inv_freq, rot_dims, norm, qkv, qkv_stride, q_weight, k_weight, eps, positions,
                                token_slot, q_out, k_cache, v_cache, page_table, table_stride_slot, table_stride_head,
                                page_size, bh_lens, T, H, G, D, Dv, reserved_slot, dtype, stream);
}

extern "C" int cvllm_bias_attn_varlen(const void* q, const void* k_cache, const void* v_cache,
                                      const int32_t* page_table, int64_t table_stride_slot, int64_t table_stride_head,
                                      int page_size, const int32_t* cu_seqlens_q, const int32_t* seq_start,
                                      const int32_t* batch_mapping, const float* slopes, int chunk, int sink,
                                      const float* sink_logits, float scale, void* out, int B, int max_new, int H, int G, int D, int Dv,
                                      int total_tokens, int64_t cache_rows, int pages_per_head, int64_t v_stride,
                                      int dtype, cvllm_stream_t stream) {
  return cvllm_bias_attn_varlen_dist(q, k_cache, v_cache, page_table, table_stride_slot, table_stride_head, page_size,
                                     cu_seqlens_q, seq_start, batch_mapping, slopes, chunk, 0, nullptr, 0, sink,
                                     sink_logits, scale, out, B, max_new, H, G, D, Dv, total_tokens, cache_rows,
                                     pages_per_head, v_stride, dtype, stream);
}

extern "C" int cvllm_bias_attn_varlen_dist(const void* q, const void* k_cache, const void* v_cache,
                                           const int32_t* page_table, int64_t table_stride_slot,
                                           int64_t table_stride_head, int page_size, const int32_t* cu_seqlens_q,
                                           const int32_t* seq_start, const int32_t* batch_mapping, const float* slopes,
                                           int chunk, int window, const float* dist_bias, int dist_rows, int sink,
                                           const float* sink_logits, float scale, void* out, int B, int max_new, int H,
                                           int G, int D, int Dv, int total_tokens, int64_t cache_rows,
                                           int pages_per_head, int64_t v_stride, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(B >= 0 && max_new >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0 && chunk >= 0);
  CVLLM_CHECK_ARG(window >= 0 && (dist_bias == nullptr || dist_rows > 0));
  const DistBias db{dist_bias, dist_rows, window};
  const bool plain_bias = window == 0 && dist_bias == nullptr;   // what the tcgen05 pipeline serves
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(q && k_cache && v_cache && page_table && cu_seqlens_q && seq_start && batch_mapping && out &&
                  check_dtype(dtype) && page_size > 0);
  CVLLM_CHECK_SUPPORTED(Dv <= 512 && B <= 65535 && H <= 65535);
  CVLLM_CHECK_ARG(v_stride == 0 || v_stride >= Dv);
  if (v_stride == 0) v_stride = Dv;
  auto st = static_cast<cudaStream_t>(stream);
  const PagedKV c = make_paged(k_cache, v_cache, page_table, table_stride_slot, table_stride_head, page_size, v_stride);
  const int64_t vec = dtype == CVLLM_BF16 ? 8 : 4;   // elements per 16-byte copy
  const int dvc = cdiv(Dv, 16);
  const float fs = sink ? 1.f : 0.f;
  const size_t cap = 226 * 1024;  // + the static row-index array
  int bn = 64;
  while (bn > 32 && varlen_smem(bn, D, Dv) > cap) bn >>= 1;
  CVLLM_CHECK_SUPPORTED(varlen_smem(bn, D, Dv) <= cap);
#define CVLLM_GO(T, BN) \
  return dispatch_dvc<T, BN>(dvc, q, c, cu_seqlens_q, seq_start, batch_mapping, slopes, chunk, db, fs, sink_logits, scale, out, B, \
                             max_new, H, G, D, Dv, st)
  const int path = test_options().bias_attn_fma.load();   // 0 product, 1 fp32 FMA kernel, 2 no tcgen05 kernel
  if (dtype == CVLLM_BF16 && D == 128 && Dv == 128 && v_stride == Dv && page_size % 128 == 0 && (H / G) % 2 == 0 &&
      path == 0 && plain_bias &&
      table_stride_head == pages_per_head && table_stride_slot == (int64_t)G * pages_per_head && cache_rows > 0)
    return cvllm_launch_prefill_bias(q, k_cache, v_cache, cache_rows, out, seq_start, slopes, page_table,
                                     batch_mapping, cu_seqlens_q, B, total_tokens, H, G, page_size, pages_per_head,
                                     max_new, scale, chunk, sink, sink_logits, st);
  if (dtype == CVLLM_BF16 && D % 16 == 0 && Dv % 8 == 0 && D <= 128 && Dv <= 128 && path != 1 &&
      v_stride % vec == 0 && aligned16(k_cache) && aligned16(v_cache)) {
    if (D <= 64 && Dv <= 64)
      return launch_varlen_mma<64>(q, c, cu_seqlens_q, seq_start, batch_mapping, slopes, chunk, db, fs, sink_logits, scale, out, B,
                                   max_new, H, G, D, Dv, st);
    return launch_varlen_mma<128>(q, c, cu_seqlens_q, seq_start, batch_mapping, slopes, chunk, db, fs, sink_logits, scale, out, B,
                                  max_new, H, G, D, Dv, st);
  }
  if (dtype == CVLLM_BF16) {
    if (bn == 64) CVLLM_GO(__nv_bfloat16, 64);
    CVLLM_GO(__nv_bfloat16, 32);
  }
  if (bn == 64) CVLLM_GO(float, 64);
  CVLLM_GO(float, 32);
#undef CVLLM_GO
}

extern "C" int cvllm_bias_attn_decode(const void* q, const void* k_cache, const void* v_cache,
                                      const int32_t* page_table, int64_t table_stride_slot, int64_t table_stride_head,
                                      int page_size, const int32_t* positions, const int32_t* batch_mapping,
                                      const float* slopes, int chunk, int sink, const float* sink_logits, float scale,
                                      void* out, int B, int H, int G, int D, int Dv, int reserved_slot, int splits, float* workspace,
                                      size_t workspace_bytes, int64_t v_stride, int dtype, cvllm_stream_t stream) {
  return cvllm_bias_attn_decode_dist(q, k_cache, v_cache, page_table, table_stride_slot, table_stride_head, page_size,
                                     positions, batch_mapping, slopes, chunk, 0, nullptr, 0, sink, sink_logits, scale,
                                     out, B, H, G, D, Dv, reserved_slot, splits, workspace, workspace_bytes, v_stride,
                                     dtype, stream);
}

extern "C" int cvllm_bias_attn_decode_dist(const void* q, const void* k_cache, const void* v_cache,
                                           const int32_t* page_table, int64_t table_stride_slot,
                                           int64_t table_stride_head, int page_size, const int32_t* positions,
                                           const int32_t* batch_mapping, const float* slopes, int chunk, int window,
                                           const float* dist_bias, int dist_rows, int sink, const float* sink_logits,
                                           float scale, void* out, int B, int H, int G, int D, int Dv,
                                           int reserved_slot, int splits, float* workspace, size_t workspace_bytes,
                                           int64_t v_stride, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(B >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0 && chunk >= 0 && splits >= 1);
  CVLLM_CHECK_ARG(window >= 0 && (dist_bias == nullptr || dist_rows > 0));
  const DistBias db{dist_bias, dist_rows, window};
  if (B == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(q && k_cache && v_cache && page_table && positions && batch_mapping && out && check_dtype(dtype) &&
                  page_size > 0);
  CVLLM_CHECK_SUPPORTED(Dv <= 32 * kDecCols && H <= 65535 && B <= 65535);
  CVLLM_CHECK_ARG(v_stride == 0 || v_stride >= Dv);
  if (v_stride == 0) v_stride = Dv;
  auto st = static_cast<cudaStream_t>(stream);
  const PagedKV c = make_paged(k_cache, v_cache, page_table, table_stride_slot, table_stride_head, page_size, v_stride);
  if (D % 8 == 0 && Dv % 8 == 0 && D <= 256 && Dv <= 256 && v_stride % 8 == 0 && aligned16(k_cache) &&
      aligned16(v_cache)) {
    if (splits > 1) {
      CVLLM_CHECK_ARG(workspace != nullptr);
      if (workspace_bytes < sizeof(float) * (size_t)B * H * splits * (2 + Dv)) {
        set_last_error("decode workspace too small");
        return CVLLM_E_WORKSPACE;
      }
    }
    const float fs = sink ? 1.f : 0.f;
    if (dtype == CVLLM_BF16)
      return launch_decode_split<__nv_bfloat16>(q, c, positions, batch_mapping, slopes, chunk, db, fs, sink_logits, scale, out,
                                                workspace, B, H, G, D, Dv, splits, reserved_slot, st);
    return launch_decode_split<float>(q, c, positions, batch_mapping, slopes, chunk, db, fs, sink_logits, scale, out, workspace, B, H,
                                      G, D, Dv, splits, reserved_slot, st);
  }
  const size_t smem = sizeof(float) * ((size_t)D + (size_t)kDecWarps * (2 + Dv));
  CVLLM_CHECK_SUPPORTED(smem <= 48 * 1024);
  dim3 grid(B, H);
  if (dtype == CVLLM_BF16)
    bias_attn_decode_kernel<__nv_bfloat16><<<grid, kDecWarps * 32, smem, st>>>(
        static_cast<const __nv_bfloat16*>(q), c, positions, batch_mapping, slopes, chunk, db, sink ? 1.f : 0.f, sink_logits, scale,
        static_cast<__nv_bfloat16*>(out), H, G, D, Dv, reserved_slot);
  else
    bias_attn_decode_kernel<float><<<grid, kDecWarps * 32, smem, st>>>(
        static_cast<const float*>(q), c, positions, batch_mapping, slopes, chunk, db, sink ? 1.f : 0.f, sink_logits, scale,
        static_cast<float*>(out), H, G, D, Dv, reserved_slot);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}
