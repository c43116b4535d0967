// Linear-attention mixers whose per-head state is a [key, value] matrix carried from token to token:
//
//   gated delta rule   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   wkv                o = (S + diag(bonus) k v^T)^T r;  S <- diag(w) S + k v^T          (w per key channel)
//   general delta rule S <- diag(w) S - (a u)(u^T S) + k v^T  (both terms on the old S);  o = S^T r
//                      (w, a per key channel, u the unit key)
//   matrix memory      m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k alone;
//                      o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)        (log gates i, f per head, capped)
//
// followed, inside the same kernel, by each head's unit norm (o / sqrt(mean(o^2) + eps)), a weight and a gate:
// out = unit(o) * norm_w * silu(gate) (or sigmoid(gate)).  Also the token shift in front of the wkv projections.
//
//   cvllm_token_shift_mix   out[s, t, :] = h_t + (h_(t-1) - h_t) * mu[s, :], the slot's last row carried between steps
//   cvllm_delta_rule        unit q / k, beta, decay, the recurrence and the gated norm
//   cvllm_wkv_scan          decays from their raw logits, the recurrence and the gated norm
//   cvllm_general_delta     unit k, removal rates, decays, the recurrence and the gated norm
//   cvllm_matrix_memory     capped log gates, the running maximum, the normalizer, the recurrence and the gated norm
//
// Geometry of a step: cu_q [B + 1] token offsets and seq_start [B] first positions of the portions, batch_mapping [B]
// slots of the state pool; cu_q == NULL means one token per sequence at positions[b] (decode steps, CUDA-graph
// replays).  A portion that starts at position 0 starts from a zero state whatever the slot holds.  States, decays,
// gates of the recurrence, norms and the outputs before the final rounding are fp32.
//
// Recurrence kernels: a cluster of one to eight CTAs per (head, sequence), the state in registers; see below.
#include <cooperative_groups.h>

#include "common.cuh"

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

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct StepGeom {
  const int32_t* cu_q;        // [B + 1] or NULL
  const int32_t* seq_start;   // [B] (with cu_q)
  const int32_t* positions;   // [B] (without cu_q)
  const int32_t* slots;       // [B]
};

__device__ __forceinline__ void portion(const StepGeom& g, int b, int& t0, int& n_new, int& start) {
  if (g.cu_q) {
    t0 = g.cu_q[b];
    n_new = g.cu_q[b + 1] - t0;
    start = g.seq_start[b];
  } else {
    t0 = b;
    n_new = 1;
    start = g.positions[b];
  }
}

// ---------------------------------------------------------------------------------------------------------
// Token shift.  grid (token tiles, B), 256 threads over the width.
// ---------------------------------------------------------------------------------------------------------
constexpr int kShiftTokens = 8;

template <typename T>
__global__ void __launch_bounds__(256) token_shift_mix_kernel(const T* __restrict__ h, int64_t h_stride,
                                                              const float* __restrict__ mu, int S, int W,
                                                              const T* __restrict__ shift_state, StepGeom g,
                                                              T* __restrict__ out, int64_t T_total) {
  const int b = blockIdx.y;
  int t0, n_new, start;
  portion(g, b, t0, n_new, start);
  const int j0 = blockIdx.x * kShiftTokens;
  if (j0 >= n_new) return;
  const int slot = g.slots[b];
  const int j1 = min(j0 + kShiftTokens, n_new);
  for (int i = threadIdx.x; i < W; i += 256) {
    float prev;
    if (j0 > 0) prev = to_f<T>(h[(int64_t)(t0 + j0 - 1) * h_stride + i]);
    else prev = start > 0 ? to_f<T>(shift_state[(int64_t)slot * W + i]) : 0.f;
    for (int j = j0; j < j1; ++j) {
      const float cur = to_f<T>(h[(int64_t)(t0 + j) * h_stride + i]);
      const float d = prev - cur;
      for (int s = 0; s < S; ++s)
        out[((int64_t)s * T_total + t0 + j) * W + i] = from_f<T>(fmaf(d, mu[(int64_t)s * W + i], cur));
      prev = cur;
    }
  }
}

// shift_state[slot] = the last row every sequence brings in this step (after the mix has read the old one)
template <typename T>
__global__ void __launch_bounds__(256) token_shift_update_kernel(const T* __restrict__ h, int64_t h_stride, int W,
                                                                 T* __restrict__ shift_state, StepGeom g,
                                                                 int reserved_slot) {
  const int b = blockIdx.x;
  int t0, n_new, start;
  portion(g, b, t0, n_new, start);
  const int slot = g.slots[b];
  if (slot == reserved_slot || n_new <= 0) return;
  for (int i = threadIdx.x; i < W; i += 256)
    shift_state[(int64_t)slot * W + i] = h[(int64_t)(t0 + n_new - 1) * h_stride + i];
}

// ---------------------------------------------------------------------------------------------------------
// Recurrences.
// A cluster of VT CTAs serves one (head, sequence): CTA v keeps value columns v * CW .. v * CW + CW - 1 of the state.
// Thread (j, s) keeps rows s * R .. s * R + R - 1 of column j in registers (KS slices of the key dimension, a power of
// two with KS * R >= D; rows beyond D stay zero), so a token costs R multiply-adds per dot product and log2(KS)
// shuffles to sum the slices.  Tokens are staged `tok` at a time in shared memory (key-sized rows in a padded slice
// layout, read as 16-byte broadcasts); the outputs of those tokens wait there for the unit norm, which runs once per
// stage with a warp per token: every CTA sums the squares of its own columns, the cluster exchanges the partial sums
// through distributed shared memory (one cluster barrier per stage, two buffers), and every CTA writes its columns.
// ---------------------------------------------------------------------------------------------------------
constexpr int kTokMax = 64;   // most tokens staged at a time (a step's count: RecurArgs::tok)

constexpr int kMaxValueDim = 256;
constexpr int kMaxKeyDim = 256;
constexpr int kMaxSlices = 32;

template <int R>
struct Lay {
  static constexpr int SL = R + 4;        // floats per slice in shared memory (the pad keeps 16-byte loads conflict-free)
  __device__ static __forceinline__ int at(int i) { return (i / R) * SL + (i % R); }
};

// sums over the KS lanes (a power of two, neighbours in the warp) that hold the slices of one value column; straight-line
// code per slice count, the two sums of slice_sum2 interleaved
__device__ __forceinline__ float slice_sum(float v, int KS) {
  switch (KS) {
    case 32: v += __shfl_xor_sync(0xffffffffu, v, 16); [[fallthrough]];
    case 16: v += __shfl_xor_sync(0xffffffffu, v, 8); [[fallthrough]];
    case 8: v += __shfl_xor_sync(0xffffffffu, v, 4); [[fallthrough]];
    case 4: v += __shfl_xor_sync(0xffffffffu, v, 2); [[fallthrough]];
    case 2: v += __shfl_xor_sync(0xffffffffu, v, 1); [[fallthrough]];
    default: break;
  }
  return v;
}

__device__ __forceinline__ void slice_sum2(float& a, float& b, int KS) {
#define CVLLM_STEP(o) a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o)
  switch (KS) {
    case 32: CVLLM_STEP(16); [[fallthrough]];
    case 16: CVLLM_STEP(8); [[fallthrough]];
    case 8: CVLLM_STEP(4); [[fallthrough]];
    case 4: CVLLM_STEP(2); [[fallthrough]];
    case 2: CVLLM_STEP(1); [[fallthrough]];
    default: break;
  }
#undef CVLLM_STEP
}

// a thread's slice (R numbers) of a staged key-sized row, as 16-byte loads into pairs (the arithmetic on the slices is
// packed: one fp32x2 instruction per two rows, each half an ordinary IEEE operation)
template <int R>
__device__ __forceinline__ void load_slice(float2 (&dst)[R / 2], const float* row_slice) {
  const float4* p = reinterpret_cast<const float4*>(row_slice);
#pragma unroll
  for (int r = 0; r < R; r += 4) {
    const float4 t = p[r / 4];
    dst[r / 2] = make_float2(t.x, t.y);
    dst[r / 2 + 1] = make_float2(t.z, t.w);
  }
}

struct RecurArgs {
  StepGeom g;
  float* state;            // [slots, H, Dv, D]: a value column's key rows are contiguous, as a thread's slice is
  const void* gate;        // [T, ..] model type: gate logits of (token, head, value channel) at gate_off + h * Dv + j
  int64_t gate_stride;
  int gate_off;
  const float* norm_w;     // weight of value channel j of head h at h * norm_head_stride + j
  int norm_head_stride;
  float eps;
  void* out;               // [T, ..] model type, head h at columns h * Dv
  int64_t out_stride;
  int H, D, Dv, reserved_slot;
  int KS, VT, CW;          // slices of the key dimension; CTAs per (head, sequence); value columns per CTA
  int tok;                 // tokens staged at a time
  int gate_kind;           // 0: silu(gate), 1: sigmoid(gate)
};

// (row, col) of the elements e = threadIdx.x + u * blockDim.x, u = 0, 1, .., of a tile [rows, width]: one division at
// the start, additions afterwards
struct TileWalk {
  int c, d, step_c, step_d, width;
  __device__ __forceinline__ TileWalk(int width_) : width(width_) {
    c = threadIdx.x / width_;
    d = threadIdx.x - c * width_;
    step_c = blockDim.x / width_;
    step_d = blockDim.x - step_c * width_;
  }
  __device__ __forceinline__ void next() {
    c += step_c;
    d += step_d;
    if (d >= width) { d -= width; ++c; }
  }
};

constexpr int kPF = 8;    // key-sized elements a thread prefetches per staged array (the rest is loaded at commit time)
constexpr int kPFG = 4;   // gate logits a thread prefetches per stage

// gate logits of the stage's (token, column) elements e = tid + u * blockDim.x, e = c * ncol + j, loaded ahead of use
template <typename T>
__device__ __forceinline__ void prefetch_gates(const RecurArgs& a, T (&pg)[kPFG], int h, int c0, int ncol, int tok0,
                                               int n) {
  const T* gate = static_cast<const T*>(a.gate);
  TileWalk w(ncol);
#pragma unroll
  for (int u = 0; u < kPFG; ++u, w.next())
    if (w.c < n) pg[u] = gate[(int64_t)(tok0 + w.c) * a.gate_stride + a.gate_off + h * a.Dv + c0 + w.d];
}

// The outputs of `n` staged tokens (so [tok][CW] fp32, this CTA's columns c0 .. c0 + ncol - 1) -> unit norm per token
// over ALL Dv columns of the head, weight, gate, rounded to the model type.  part [2][kTokMax]: this CTA's sums of squares,
// read by the other CTAs of the cluster (`stage` picks the buffer); sinv [kTokMax]: the tokens' 1 / rms.  Every CTA of the
// cluster calls this the same number of times (they share the sequence), so the cluster barrier inside is matched.
template <typename T>
__device__ __forceinline__ void gated_unit_norm_rows(const RecurArgs& a, const float* so, float* part, float* sinv,
                                                     int stage, const T (&pg)[kPFG], int h, int c0, int ncol, int tok0,
                                                     int n) {
  namespace cg = cooperative_groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const T* gate = static_cast<const T*>(a.gate);
  T* out = static_cast<T*>(a.out);
  float* mine = part + (stage & 1) * kTokMax;
  for (int c = warp; c < n; c += warps) {
    const float* o = so + c * a.CW;
    float ss = 0.f;
    for (int j = lane; j < ncol; j += 32) ss += o[j] * o[j];
    ss = warp_sum(ss);
    if (lane == 0) mine[c] = ss;
  }
  if (a.VT > 1) cg::this_cluster().sync();
  else __syncthreads();
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float ss = 0.f;
    if (a.VT > 1) {
      cg::cluster_group cl = cg::this_cluster();
      for (int v = 0; v < a.VT; ++v) ss += cl.map_shared_rank(mine, v)[c];
    } else {
      ss = mine[c];
    }
    sinv[c] = 1.0f / sqrtf(ss / (float)a.Dv + a.eps);
  }
  __syncthreads();
  auto emit = [&](int c, int j, float gz) {
    const int col = h * a.Dv + c0 + j;
    out[(int64_t)(tok0 + c) * a.out_stride + col] =
        from_f<T>(so[c * a.CW + j] * sinv[c] * a.norm_w[h * a.norm_head_stride + c0 + j] *
                  (a.gate_kind ? sigmoid_f(gz) : silu_f(gz)));
  };
  TileWalk w(ncol);
#pragma unroll
  for (int u = 0; u < kPFG; ++u, w.next())
    if (w.c < n) emit(w.c, w.d, to_f<T>(pg[u]));
  for (; w.c < n; w.next())
    emit(w.c, w.d, to_f<T>(gate[(int64_t)(tok0 + w.c) * a.gate_stride + a.gate_off + h * a.Dv + c0 + w.d]));
}

// State of (slot, head): [Dv, D] fp32, the key rows of a value column contiguous - a thread's slice is R consecutive
// numbers, moved as 16-byte pieces when the key size allows.
template <int R>
__device__ __forceinline__ void load_state(float2 (&S)[R / 2], const RecurArgs& a, int slot, int h, int col, bool valid,
                                           int ks, bool from_pool) {
  const float* src = a.state + (((int64_t)slot * a.H + h) * a.Dv + col) * a.D;
  const bool on = from_pool && valid;
  if ((a.D & 3) == 0) {
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      const int i = ks * R + r;
      float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
      if (on && i < a.D) t = *reinterpret_cast<const float4*>(src + i);
      S[r / 2] = make_float2(t.x, t.y);
      S[r / 2 + 1] = make_float2(t.z, t.w);
    }
  } else {
#pragma unroll
    for (int r = 0; r < R; r += 2) {
      const int i = ks * R + r;
      S[r / 2] = make_float2((on && i < a.D) ? src[i] : 0.f, (on && i + 1 < a.D) ? src[i + 1] : 0.f);
    }
  }
}

template <int R>
__device__ __forceinline__ void store_state(const float2 (&S)[R / 2], const RecurArgs& a, int slot, int h, int col,
                                            bool valid, int ks) {
  float* dst = a.state + (((int64_t)slot * a.H + h) * a.Dv + col) * a.D;
  if ((a.D & 3) == 0) {
#pragma unroll
    for (int r = 0; r < R; r += 4) {
      const int i = ks * R + r;
      if (valid && i < a.D)
        *reinterpret_cast<float4*>(dst + i) = make_float4(S[r / 2].x, S[r / 2].y, S[r / 2 + 1].x, S[r / 2 + 1].y);
    }
  } else {
#pragma unroll
    for (int r = 0; r < R; r += 2) {
      const int i = ks * R + r;
      if (valid && i < a.D) dst[i] = S[r / 2].x;
      if (valid && i + 1 < a.D) dst[i + 1] = S[r / 2].y;
    }
  }
}

// Gated delta rule.  qkv [T, 2 G D + H Dv] fp32 = (q | k | v) after the short convolution; beta and decay logits are
// columns b_off + h and a_off + h of proj (model type).  Head h reads q / k head h / (H / G).
// Algebra per token, from the state S before the token:  dk = S^T k, dq = S^T q (one pass over the registers),
// u = beta (v - g dk),  o = g dq + (k . q) u,  S <- g S + k u^T   - the same numbers as decaying first, writing, then
// reading, with one pass less over the state.
template <typename T, int R, int MAXT>
__global__ void __launch_bounds__(MAXT) delta_rule_kernel(const float* __restrict__ qkv, int64_t qkv_stride,
                                                          const T* __restrict__ proj, int64_t proj_stride, int b_off,
                                                          int a_off, const float* __restrict__ A_log,
                                                          const float* __restrict__ dt_bias, int G, RecurArgs a) {
  using L = Lay<R>;
  extern __shared__ __align__(16) float sm[];
  const int D = a.D, Dv = a.Dv, H = a.H, KS = a.KS, CW = a.CW, kTok = a.tok;
  const int ROW = KS * L::SL;
  float* sq = sm;                       // [kTok][ROW]
  float* sk = sq + kTok * ROW;          // [kTok][ROW]
  float* sv = sk + kTok * ROW;          // [kTok][CW]
  float* so = sv + kTok * CW;           // [kTok][CW]
  float* sc = so + kTok * CW;           // [kTok][4]: decay, beta, k . q
  float* part = sc + kTok * 4;          // [2][kTokMax]
  float* sinv = part + 2 * kTokMax;     // [kTokMax]
  const int h = blockIdx.x / a.VT, vt = blockIdx.x % a.VT, b = blockIdx.y;
  int t0, n_new, start;
  portion(a.g, b, t0, n_new, start);
  if (n_new <= 0) return;               // the same for every CTA of the cluster
  const int slot = a.g.slots[b];
  const int kvh = h / (H / G);
  const int c0 = vt * CW, ncol = min(CW, Dv - c0);
  const int tid = threadIdx.x, j = tid / KS, ks = tid % KS;
  const bool valid = j < ncol;
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
  for (int i = tid; i < 2 * kTok * ROW; i += blockDim.x) sm[i] = 0.f;   // pads and rows beyond D stay zero
  float2 S[R / 2];
  load_state<R>(S, a, slot, h, c0 + j, valid, ks, start > 0);
  const float neg_a = -expf(A_log[h]), dtb = dt_bias[h];
  const float q_scale = rsqrtf((float)D);
  const int q_col = kvh * D, k_col = G * D + kvh * D, v_col = 2 * G * D + h * Dv + c0;
  __syncthreads();
  // a stage's inputs are loaded into registers one stage ahead, so that their latency hides behind the tokens before
  float pq[kPF], pk[kPF], pv[kPFG];
  T pg[kPFG];
  auto prefetch = [&](int j0n) {
    const int nn = min(kTok, n_new - j0n);
    TileWalk w(D);
#pragma unroll
    for (int u = 0; u < kPF; ++u, w.next())
      if (w.c < nn) {
        const float* row = qkv + (int64_t)(t0 + j0n + w.c) * qkv_stride;
        pq[u] = row[q_col + w.d];
        pk[u] = row[k_col + w.d];
      }
    TileWalk wv(ncol);
#pragma unroll
    for (int u = 0; u < kPFG; ++u, wv.next())
      if (wv.c < nn) pv[u] = qkv[(int64_t)(t0 + j0n + wv.c) * qkv_stride + v_col + wv.d];
  };
  prefetch(0);
  int stage = 0;
  for (int j0 = 0; j0 < n_new; j0 += kTok, ++stage) {
    const int n = min(kTok, n_new - j0);
    {
      TileWalk w(D);
#pragma unroll
      for (int u = 0; u < kPF; ++u, w.next())
        if (w.c < n) {
          sq[w.c * ROW + L::at(w.d)] = pq[u];
          sk[w.c * ROW + L::at(w.d)] = pk[u];
        }
      for (; w.c < n; w.next()) {
        const float* row = qkv + (int64_t)(t0 + j0 + w.c) * qkv_stride;
        sq[w.c * ROW + L::at(w.d)] = row[q_col + w.d];
        sk[w.c * ROW + L::at(w.d)] = row[k_col + w.d];
      }
      TileWalk wv(ncol);
#pragma unroll
      for (int u = 0; u < kPFG; ++u, wv.next())
        if (wv.c < n) sv[wv.c * CW + wv.d] = pv[u];
      for (; wv.c < n; wv.next()) sv[wv.c * CW + wv.d] = qkv[(int64_t)(t0 + j0 + wv.c) * qkv_stride + v_col + wv.d];
    }
    for (int c = tid; c < n; c += blockDim.x) {   // the tokens' decays and betas
      const T* pr = proj + (int64_t)(t0 + j0 + c) * proj_stride;
      sc[c * 4 + 0] = expf(neg_a * softplus_f(to_f<T>(pr[a_off + h]) + dtb));
      sc[c * 4 + 1] = sigmoid_f(to_f<T>(pr[b_off + h]));
    }
    __syncthreads();
    if (j0 + kTok < n_new) prefetch(j0 + kTok);
    prefetch_gates<T>(a, pg, h, c0, ncol, t0 + j0, n);
    for (int c = warp; c < n; c += warps) {   // unit q and k, the token's scalars
      float qq = 0.f, kk = 0.f, qk = 0.f;
      for (int d = lane; d < D; d += 32) {
        const float qv = sq[c * ROW + L::at(d)], kv = sk[c * ROW + L::at(d)];
        qq += qv * qv;
        kk += kv * kv;
        qk += qv * kv;
      }
      qq = warp_sum(qq);
      kk = warp_sum(kk);
      qk = warp_sum(qk);
      const float qi = q_scale / sqrtf(qq + 1e-6f), ki = 1.0f / sqrtf(kk + 1e-6f);
      for (int d = lane; d < D; d += 32) {
        sq[c * ROW + L::at(d)] *= qi;
        sk[c * ROW + L::at(d)] *= ki;
      }
      if (lane == 0) sc[c * 4 + 2] = qk * qi * ki;
    }
    __syncthreads();
    // One token: its key / query slices are in registers already (loaded while the token before ran); the next token's
    // are requested first.  Four partial sums per dot product keep the multiply-add chains short.
    auto step = [&](const float2 (&kc)[R / 2], const float2 (&qc)[R / 2], float2 (&kn)[R / 2], float2 (&qn)[R / 2], int c,
                    bool ahead) {
      if (ahead && c + 1 < n) {
        load_slice<R>(kn, sk + (c + 1) * ROW + ks * L::SL);
        load_slice<R>(qn, sq + (c + 1) * ROW + ks * L::SL);
      }
      const float gd = sc[c * 4 + 0], beta = sc[c * 4 + 1], kq_dot = sc[c * 4 + 2];
      const float vj = valid ? sv[c * CW + j] : 0.f;
      float2 dk[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)}, dq[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int r = 0; r < R / 2; ++r) {
        dk[r & 1] = __ffma2_rn(S[r], kc[r], dk[r & 1]);
        dq[r & 1] = __ffma2_rn(S[r], qc[r], dq[r & 1]);
      }
      float dks = (dk[0].x + dk[0].y) + (dk[1].x + dk[1].y), dqs = (dq[0].x + dq[0].y) + (dq[1].x + dq[1].y);
      slice_sum2(dks, dqs, KS);
      const float u = beta * (vj - gd * dks);
      if (ks == 0 && valid) so[c * CW + j] = fmaf(kq_dot, u, gd * dqs);
      const float2 u2 = make_float2(u, u), g2 = make_float2(gd, gd);
#pragma unroll
      for (int r = 0; r < R / 2; ++r) S[r] = __ffma2_rn(kc[r], u2, __fmul2_rn(g2, S[r]));
    };
    if constexpr (R <= 16) {
      float2 ka[R / 2], qa[R / 2], kb[R / 2], qb[R / 2];
      load_slice<R>(ka, sk + ks * L::SL);
      load_slice<R>(qa, sq + ks * L::SL);
      for (int c = 0; c < n; c += 2) {
        step(ka, qa, kb, qb, c, true);
        if (c + 1 < n) step(kb, qb, ka, qa, c + 1, true);
      }
    } else {   // long slices: no registers to spare for the token ahead
      float2 ka[R / 2], qa[R / 2];
      for (int c = 0; c < n; ++c) {
        load_slice<R>(ka, sk + c * ROW + ks * L::SL);
        load_slice<R>(qa, sq + c * ROW + ks * L::SL);
        step(ka, qa, ka, qa, c, false);
      }
    }
    __syncthreads();
    gated_unit_norm_rows<T>(a, so, part, sinv, stage, pg, h, c0, ncol, t0 + j0, n);
    __syncthreads();
  }
  if (slot != a.reserved_slot) store_state<R>(S, a, slot, h, c0 + j, valid, ks);
  if (a.VT > 1) cooperative_groups::this_cluster().sync();   // nobody leaves while its sums may still be read
}

// wkv.  r, k, v: [T, H * D] rows of the model type (row strides given); w_raw [T, H * D] decay logits (model type):
// w = exp(-exp(w_raw + w0)); bonus [H * D] multiplies the current token's own k v^T in its read-out only.  Dv = D.
template <typename T, int R, int MAXT>
__global__ void __launch_bounds__(MAXT) wkv_scan_kernel(const T* __restrict__ rp, int64_t r_stride,
                                                        const T* __restrict__ kp, int64_t k_stride,
                                                        const T* __restrict__ vp, int64_t v_stride,
                                                        const T* __restrict__ wp, int64_t w_stride,
                                                        const float* __restrict__ w0, const float* __restrict__ bonus,
                                                        RecurArgs a) {
  using L = Lay<R>;
  extern __shared__ __align__(16) float sm[];
  const int D = a.D, Dv = a.Dv, KS = a.KS, CW = a.CW, kTok = a.tok;
  const int ROW = KS * L::SL;
  float* sr = sm;                       // [kTok][ROW]
  float* sk = sr + kTok * ROW;          // [kTok][ROW]
  float* sw = sk + kTok * ROW;          // [kTok][ROW]
  float* sv = sw + kTok * ROW;          // [kTok][CW]
  float* so = sv + kTok * CW;           // [kTok][CW]
  float* part = so + kTok * CW;         // [2][kTokMax]
  float* sinv = part + 2 * kTokMax;     // [kTokMax]
  float* sc = sinv + kTokMax;           // [kTokMax]: sum_i r_i bonus_i k_i of the token
  const int h = blockIdx.x / a.VT, vt = blockIdx.x % a.VT, b = blockIdx.y;
  int t0, n_new, start;
  portion(a.g, b, t0, n_new, start);
  if (n_new <= 0) return;               // the same for every CTA of the cluster
  const int slot = a.g.slots[b];
  const int c0 = vt * CW, ncol = min(CW, Dv - c0);
  const int tid = threadIdx.x, j = tid / KS, ks = tid % KS;
  const bool valid = j < ncol;
  for (int i = tid; i < 3 * kTok * ROW; i += blockDim.x) sm[i] = 0.f;   // pads and rows beyond D stay zero
  float2 S[R / 2];
  load_state<R>(S, a, slot, h, c0 + j, valid, ks, start > 0);
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
  __syncthreads();
  // a stage's inputs are loaded into registers one stage ahead, so that their latency hides behind the tokens before
  T pr_[kPF], pk_[kPF], pw_[kPF], pv_[kPFG], pg[kPFG];
  auto prefetch = [&](int j0n) {
    const int nn = min(kTok, n_new - j0n);
    TileWalk w(D);
#pragma unroll
    for (int u = 0; u < kPF; ++u, w.next())
      if (w.c < nn) {
        const int64_t t = t0 + j0n + w.c;
        const int col = h * D + w.d;
        pr_[u] = rp[t * r_stride + col];
        pk_[u] = kp[t * k_stride + col];
        pw_[u] = wp[t * w_stride + col];
      }
    TileWalk wv(ncol);
#pragma unroll
    for (int u = 0; u < kPFG; ++u, wv.next())
      if (wv.c < nn) pv_[u] = vp[(int64_t)(t0 + j0n + wv.c) * v_stride + h * Dv + c0 + wv.d];
  };
  prefetch(0);
  int stage = 0;
  for (int j0 = 0; j0 < n_new; j0 += kTok, ++stage) {
    const int n = min(kTok, n_new - j0);
    {
      TileWalk w(D);
#pragma unroll
      for (int u = 0; u < kPF; ++u, w.next())
        if (w.c < n) {
          sr[w.c * ROW + L::at(w.d)] = to_f<T>(pr_[u]);
          sk[w.c * ROW + L::at(w.d)] = to_f<T>(pk_[u]);
          sw[w.c * ROW + L::at(w.d)] = expf(-expf(to_f<T>(pw_[u]) + w0[h * D + w.d]));
        }
      for (; w.c < n; w.next()) {
        const int64_t t = t0 + j0 + w.c;
        const int col = h * D + w.d;
        sr[w.c * ROW + L::at(w.d)] = to_f<T>(rp[t * r_stride + col]);
        sk[w.c * ROW + L::at(w.d)] = to_f<T>(kp[t * k_stride + col]);
        sw[w.c * ROW + L::at(w.d)] = expf(-expf(to_f<T>(wp[t * w_stride + col]) + w0[col]));
      }
      TileWalk wv(ncol);
#pragma unroll
      for (int u = 0; u < kPFG; ++u, wv.next())
        if (wv.c < n) sv[wv.c * CW + wv.d] = to_f<T>(pv_[u]);
      for (; wv.c < n; wv.next())
        sv[wv.c * CW + wv.d] = to_f<T>(vp[(int64_t)(t0 + j0 + wv.c) * v_stride + h * Dv + c0 + wv.d]);
    }
    __syncthreads();
    if (j0 + kTok < n_new) prefetch(j0 + kTok);
    prefetch_gates<T>(a, pg, h, c0, ncol, t0 + j0, n);
    // the bonus acts on the token's own k v^T only:  (diag(bonus) k v^T)^T r = v * sum_i r_i bonus_i k_i, one number a token
    for (int c = warp; c < n; c += warps) {
      float acc = 0.f;
      for (int d = lane; d < D; d += 32) acc += sr[c * ROW + L::at(d)] * bonus[h * D + d] * sk[c * ROW + L::at(d)];
      acc = warp_sum(acc);
      if (lane == 0) sc[c] = acc;
    }
    __syncthreads();
    // One token: its r / k / w slices are in registers already (loaded while the token before ran); the next token's
    // are requested first.  The read-out uses the state BEFORE the token's write; four partial sums keep its chain short.
    auto step = [&](const float2 (&rc)[R / 2], const float2 (&kc)[R / 2], const float2 (&wc)[R / 2], float2 (&rn)[R / 2],
                    float2 (&kn)[R / 2], float2 (&wn)[R / 2], int c, bool ahead) {
      if (ahead && c + 1 < n) {
        load_slice<R>(rn, sr + (c + 1) * ROW + ks * L::SL);
        load_slice<R>(kn, sk + (c + 1) * ROW + ks * L::SL);
        load_slice<R>(wn, sw + (c + 1) * ROW + ks * L::SL);
      }
      const float vj = valid ? sv[c * CW + j] : 0.f;
      const float own = sc[c];
      float2 o[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int r = 0; r < R / 2; ++r) {
        o[r & 1].x = fmaf(rc[r].x, S[r].x, o[r & 1].x);
        o[r & 1].y = fmaf(rc[r].y, S[r].y, o[r & 1].y);
        S[r].x = fmaf(wc[r].x, S[r].x, kc[r].x * vj);
        S[r].y = fmaf(wc[r].y, S[r].y, kc[r].y * vj);
      }
      const float os = slice_sum((o[0].x + o[0].y) + (o[1].x + o[1].y), KS);
      if (ks == 0 && valid) so[c * CW + j] = fmaf(vj, own, os);
    };
    if constexpr (R <= 8) {
      float2 ra[R / 2], ka[R / 2], wa[R / 2], rb[R / 2], kb[R / 2], wb[R / 2];
      load_slice<R>(ra, sr + ks * L::SL);
      load_slice<R>(ka, sk + ks * L::SL);
      load_slice<R>(wa, sw + ks * L::SL);
      for (int c = 0; c < n; c += 2) {
        step(ra, ka, wa, rb, kb, wb, c, true);
        if (c + 1 < n) step(rb, kb, wb, ra, ka, wa, c + 1, true);
      }
    } else {   // long slices: no registers to spare for the token ahead
      float2 ra[R / 2], ka[R / 2], wa[R / 2];
      for (int c = 0; c < n; ++c) {
        load_slice<R>(ra, sr + c * ROW + ks * L::SL);
        load_slice<R>(ka, sk + c * ROW + ks * L::SL);
        load_slice<R>(wa, sw + c * ROW + ks * L::SL);
        step(ra, ka, wa, ra, ka, wa, c, false);
      }
    }
    __syncthreads();
    gated_unit_norm_rows<T>(a, so, part, sinv, stage, pg, h, c0, ncol, t0 + j0, n);
    __syncthreads();
  }
  if (slot != a.reserved_slot) store_state<R>(S, a, slot, h, c0 + j, valid, ks);
  if (a.VT > 1) cooperative_groups::this_cluster().sync();   // nobody leaves while its sums may still be read
}

// General delta rule.  r, k, v, the removal-rate logits (a) and the gate are columns of proj (model type) at r_off,
// k_off, v_off, a_off (+ h * D) and gate_off; w_raw [T, H * D] decay logits: w = exp(-rate * sigmoid(w_raw + w0)).
// Dv = D.  With u = k / sqrt(sum k^2 + 1e-6) and au = sigmoid(a) u, per value column j from the column s before the token:
//   d1 = u . s,  d2 = (r w) . s   (one pass),   o_j = d2 - (r . au) d1 + (r . k) v_j,   s <- w s - au d1 + k v_j
// - the numbers of "decay, remove, write, then read" with one pass over the state for both dot products.
template <typename T, int R, int MAXT>
__global__ void __launch_bounds__(MAXT) general_delta_kernel(const T* __restrict__ proj, int64_t proj_stride, int r_off,
                                                             int k_off, int v_off, int a_off,
                                                             const T* __restrict__ wp, int64_t w_stride,
                                                             const float* __restrict__ w0, float rate, RecurArgs a) {
  using L = Lay<R>;
  extern __shared__ __align__(16) float sm[];
  const int D = a.D, Dv = a.Dv, KS = a.KS, CW = a.CW, kTok = a.tok;
  const int ROW = KS * L::SL;
  float* su = sm;                       // [kTok][ROW] unit keys
  float* sy = su + kTok * ROW;          // [kTok][ROW] r * w
  float* sw = sy + kTok * ROW;          // [kTok][ROW] w
  float* sa = sw + kTok * ROW;          // [kTok][ROW] sigmoid(a) * u
  float* sk = sa + kTok * ROW;          // [kTok][ROW] k
  float* sv = sk + kTok * ROW;          // [kTok][CW]
  float* so = sv + kTok * CW;           // [kTok][CW]
  float* sc = so + kTok * CW;           // [kTok][4]: r . au, r . k
  float* part = sc + kTok * 4;          // [2][kTokMax]
  float* sinv = part + 2 * kTokMax;     // [kTokMax]
  const int h = blockIdx.x / a.VT, vt = blockIdx.x % a.VT, b = blockIdx.y;
  int t0, n_new, start;
  portion(a.g, b, t0, n_new, start);
  if (n_new <= 0) return;               // the same for every CTA of the cluster
  const int slot = a.g.slots[b];
  const int c0 = vt * CW, ncol = min(CW, Dv - c0);
  const int tid = threadIdx.x, j = tid / KS, ks = tid % KS;
  const bool valid = j < ncol;
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
  for (int i = tid; i < 5 * kTok * ROW; i += blockDim.x) sm[i] = 0.f;   // pads and rows beyond D stay zero
  float2 S[R / 2];
  load_state<R>(S, a, slot, h, c0 + j, valid, ks, start > 0);
  T pg[kPFG];
  __syncthreads();
  int stage = 0;
  for (int j0 = 0; j0 < n_new; j0 += kTok, ++stage) {
    const int n = min(kTok, n_new - j0);
    {   // the stage's raw rows, all threads: k, r, the removal-rate logits and the decay logits land in their planes
      TileWalk w(D);
      for (; w.c < n; w.next()) {
        const T* pr = proj + (int64_t)(t0 + j0 + w.c) * proj_stride + h * D;
        const int at = w.c * ROW + L::at(w.d);
        sk[at] = to_f<T>(pr[k_off + w.d]);
        sy[at] = to_f<T>(pr[r_off + w.d]);
        sa[at] = to_f<T>(pr[a_off + w.d]);
        sw[at] = to_f<T>(wp[(int64_t)(t0 + j0 + w.c) * w_stride + h * D + w.d]);
      }
    }
    for (int i = tid; i < n * ncol; i += blockDim.x) {
      const int c = i / ncol, d = i - c * ncol;
      sv[c * CW + d] = to_f<T>(proj[(int64_t)(t0 + j0 + c) * proj_stride + v_off + h * Dv + c0 + d]);
    }
    __syncthreads();
    for (int c = warp; c < n; c += warps) {   // a warp per token: unit key, rates, decays, the token's two scalars
      float kk = 0.f;
      for (int d = lane; d < D; d += 32) {
        const float kv = sk[c * ROW + L::at(d)];
        kk += kv * kv;
      }
      kk = warp_sum(kk);
      const float ki = 1.0f / sqrtf(kk + 1e-6f);
      float rau = 0.f, rk = 0.f;
      for (int d = lane; d < D; d += 32) {
        const int at = c * ROW + L::at(d);
        const float kv = sk[at], rv = sy[at];
        const float u = kv * ki, au = sigmoid_f(sa[at]) * u;
        const float w = exp_1ulp(-rate * sigmoid_f(sw[at] + w0[h * D + d]));   // multiplies the state token after token
        su[at] = u;
        sy[at] = rv * w;
        sw[at] = w;
        sa[at] = au;
        rau = fmaf(rv, au, rau);
        rk = fmaf(rv, kv, rk);
      }
      rau = warp_sum(rau);
      rk = warp_sum(rk);
      if (lane == 0) {
        sc[c * 4 + 0] = rau;
        sc[c * 4 + 1] = rk;
      }
    }
    prefetch_gates<T>(a, pg, h, c0, ncol, t0 + j0, n);
    __syncthreads();
    for (int c = 0; c < n; ++c) {
      const float vj = valid ? sv[c * CW + j] : 0.f;
      const float* base = sm + c * ROW + ks * L::SL;
      const int plane = kTok * ROW;
      float2 d1[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)}, d2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 u4 = *reinterpret_cast<const float4*>(base + r);
        const float4 y4 = *reinterpret_cast<const float4*>(base + plane + r);
        d1[0] = __ffma2_rn(S[r / 2], make_float2(u4.x, u4.y), d1[0]);
        d1[1] = __ffma2_rn(S[r / 2 + 1], make_float2(u4.z, u4.w), d1[1]);
        d2[0] = __ffma2_rn(S[r / 2], make_float2(y4.x, y4.y), d2[0]);
        d2[1] = __ffma2_rn(S[r / 2 + 1], make_float2(y4.z, y4.w), d2[1]);
      }
      float d1s = (d1[0].x + d1[0].y) + (d1[1].x + d1[1].y), d2s = (d2[0].x + d2[0].y) + (d2[1].x + d2[1].y);
      slice_sum2(d1s, d2s, KS);
      if (ks == 0 && valid) so[c * CW + j] = fmaf(sc[c * 4 + 1], vj, fmaf(-sc[c * 4 + 0], d1s, d2s));
      const float2 nd = make_float2(-d1s, -d1s), v2 = make_float2(vj, vj);
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 w4 = *reinterpret_cast<const float4*>(base + 2 * plane + r);
        const float4 a4 = *reinterpret_cast<const float4*>(base + 3 * plane + r);
        const float4 k4 = *reinterpret_cast<const float4*>(base + 4 * plane + r);
        float2 x0 = __fmul2_rn(make_float2(w4.x, w4.y), S[r / 2]);
        float2 x1 = __fmul2_rn(make_float2(w4.z, w4.w), S[r / 2 + 1]);
        x0 = __ffma2_rn(make_float2(a4.x, a4.y), nd, x0);
        x1 = __ffma2_rn(make_float2(a4.z, a4.w), nd, x1);
        S[r / 2] = __ffma2_rn(make_float2(k4.x, k4.y), v2, x0);
        S[r / 2 + 1] = __ffma2_rn(make_float2(k4.z, k4.w), v2, x1);
      }
    }
    __syncthreads();
    gated_unit_norm_rows<T>(a, so, part, sinv, stage, pg, h, c0, ncol, t0 + j0, n);
    __syncthreads();
  }
  if (slot != a.reserved_slot) store_state<R>(S, a, slot, h, c0 + j, valid, ks);
  if (a.VT > 1) cooperative_groups::this_cluster().sync();   // nobody leaves while its sums may still be read
}

// Matrix memory with exponential gates kept in range by a running maximum.  q, k, v, the gate and the two log-gate
// logits (one per head) are columns of proj (model type) at q_off, k_off (+ h * D), v_off, gate_off (+ h * Dv),
// i_off + h and f_off + h (biases already added).  i = cap tanh(z_i / cap), f = logsigmoid(cap tanh(z_f / cap));
// m' = max(f + m, i), F = exp(f + m - m'), I = exp(i - m');  n <- F n + I k;  per value column j from the column s
// before the token:  d = s . q,  o_j = (F d + I (k . q) v_j) / (max(|n . q|, exp(-m')) + 1e-6),  s <- F s + I v_j k.
// q carries q_scale.  The running maximum m starts at 0, n and S at zero; nvec [slots, H, D] and mstate [slots, H]
// hold n and m between steps.  The normalizer n is the state's column of a value that is always 1: every CTA keeps it
// as one more column (threads j == ncol) and gets n . q from the same pass as its read-outs; the division waits for
// the end of the stage.  The maximum and the two gates are a scalar recurrence over the tokens: the CTA's LAST warp
// has no columns and walks it for the NEXT stage while the other warps run the current stage's tokens; a stage's
// inputs are loaded into registers one stage ahead, as in the delta rule.
template <typename T, int R, int MAXT>
__global__ void __launch_bounds__(MAXT) matrix_memory_kernel(const T* __restrict__ proj, int64_t proj_stride, int q_off,
                                                             int k_off, int v_off, int i_off, int f_off, float cap,
                                                             float q_scale, float* __restrict__ nvec,
                                                             float* __restrict__ mstate, RecurArgs a) {
  using L = Lay<R>;
  extern __shared__ __align__(16) float sm[];
  const int D = a.D, Dv = a.Dv, H = a.H, KS = a.KS, CW = a.CW, kTok = a.tok;
  const int ROW = KS * L::SL;
  float* sq = sm;                       // [kTok][ROW]
  float* sk = sq + kTok * ROW;          // [kTok][ROW]
  float* sv = sk + kTok * ROW;          // [kTok][CW]
  float* so = sv + kTok * CW;           // [kTok][CW]
  float* skq = so + kTok * CW;          // [kTok][4]: k . q of the token (first of four)
  float* part = skq + kTok * 4;         // [2][kTokMax]
  float* sinv = part + 2 * kTokMax;     // [kTokMax]
  float* sden = sinv + kTokMax;         // [kTokMax]: n . q of the token
  float* sg = sden + kTokMax;           // [2][kTokMax][4]: per stage parity: F, I, exp(-m') (before the walk: f, i)
  const int h = blockIdx.x / a.VT, vt = blockIdx.x % a.VT, b = blockIdx.y;
  int t0, n_new, start;
  portion(a.g, b, t0, n_new, start);
  if (n_new <= 0) return;               // the same for every CTA of the cluster
  const int slot = a.g.slots[b];
  const int c0 = vt * CW, ncol = min(CW, Dv - c0);
  const int tid = threadIdx.x, j = tid / KS, ks = tid % KS;
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
  const int workers = warps - 1;        // warps with columns; the last warp walks the gates
  const bool walker_warp = warp == workers;
  const bool valid = j < ncol && !walker_warp, is_n = j == ncol && !walker_warp;
  const int wthreads = workers * 32;
  for (int i = tid; i < 2 * kTok * ROW; i += blockDim.x) sm[i] = 0.f;   // pads and rows beyond D stay zero
  float2 S[R / 2];
  load_state<R>(S, a, slot, h, c0 + j, valid, ks, start > 0);
  if (is_n) {
    const float* src = nvec + ((int64_t)slot * H + h) * D;
#pragma unroll
    for (int r = 0; r < R; r += 2) {
      const int i = ks * R + r;
      S[r / 2] = make_float2((start > 0 && i < D) ? src[i] : 0.f, (start > 0 && i + 1 < D) ? src[i + 1] : 0.f);
    }
  }
  float mrun = (walker_warp && lane == 0 && start > 0) ? mstate[(int64_t)slot * H + h] : 0.f;
  // the capped log gates of a stage's tokens (any thread may make them), then the walk by one lane
  auto gates = [&](int j0n, float* dst) {
    const int nn = min(kTok, n_new - j0n);
    for (int c = tid; c < nn; c += blockDim.x) {
      const T* pr = proj + (int64_t)(t0 + j0n + c) * proj_stride;
      const float zi = cap * tanhf(to_f<T>(pr[i_off + h]) / cap), zf = cap * tanhf(to_f<T>(pr[f_off + h]) / cap);
      dst[c * 4 + 0] = zf < -20.f ? zf : -log1pf(expf(-zf));   // logsigmoid
      dst[c * 4 + 1] = zi;
    }
  };
  auto walk = [&](int j0n, float* dst) {
    const int nn = min(kTok, n_new - j0n);
    for (int c = 0; c < nn; ++c) {
      const float fl = dst[c * 4 + 0], il = dst[c * 4 + 1];
      const float m_new = fmaxf(fl + mrun, il);
      dst[c * 4 + 0] = exp_1ulp(fl + mrun - m_new);     // the state's factor, token after token
      dst[c * 4 + 1] = exp_1ulp(il - m_new);
      dst[c * 4 + 2] = expf(-m_new);
      mrun = m_new;
    }
  };
  T pq[kPF], pk[kPF], pv[kPFG], pg[kPFG];
  auto prefetch = [&](int j0n) {
    const int nn = min(kTok, n_new - j0n);
    TileWalk w(D);
#pragma unroll
    for (int u = 0; u < kPF; ++u, w.next())
      if (w.c < nn) {
        const T* pr = proj + (int64_t)(t0 + j0n + w.c) * proj_stride + h * D;
        pq[u] = pr[q_off + w.d];
        pk[u] = pr[k_off + w.d];
      }
    TileWalk wv(ncol);
#pragma unroll
    for (int u = 0; u < kPFG; ++u, wv.next())
      if (wv.c < nn) pv[u] = proj[(int64_t)(t0 + j0n + wv.c) * proj_stride + v_off + h * Dv + c0 + wv.d];
  };
  prefetch(0);
  gates(0, sg);
  __syncthreads();
  if (walker_warp && lane == 0) walk(0, sg);
  int stage = 0;
  for (int j0 = 0; j0 < n_new; j0 += kTok, ++stage) {
    const int n = min(kTok, n_new - j0);
    float* cur = sg + (stage & 1) * kTokMax * 4;
    float* nxt = sg + ((stage + 1) & 1) * kTokMax * 4;
    {
      TileWalk w(D);
#pragma unroll
      for (int u = 0; u < kPF; ++u, w.next())
        if (w.c < n) {
          sq[w.c * ROW + L::at(w.d)] = to_f<T>(pq[u]) * q_scale;
          sk[w.c * ROW + L::at(w.d)] = to_f<T>(pk[u]);
        }
      for (; w.c < n; w.next()) {
        const T* pr = proj + (int64_t)(t0 + j0 + w.c) * proj_stride + h * D;
        sq[w.c * ROW + L::at(w.d)] = to_f<T>(pr[q_off + w.d]) * q_scale;
        sk[w.c * ROW + L::at(w.d)] = to_f<T>(pr[k_off + w.d]);
      }
      TileWalk wv(ncol);
#pragma unroll
      for (int u = 0; u < kPFG; ++u, wv.next())
        if (wv.c < n) sv[wv.c * CW + wv.d] = to_f<T>(pv[u]);
      for (; wv.c < n; wv.next())
        sv[wv.c * CW + wv.d] = to_f<T>(proj[(int64_t)(t0 + j0 + wv.c) * proj_stride + v_off + h * Dv + c0 + wv.d]);
    }
    if (j0 + kTok < n_new) gates(j0 + kTok, nxt);
    __syncthreads();                    // the stage's rows, this stage's walked gates and the next stage's raw gates are in place
    if (j0 + kTok < n_new) prefetch(j0 + kTok);
    prefetch_gates<T>(a, pg, h, c0, ncol, t0 + j0, n);
    if (walker_warp) {
      if (lane == 0 && j0 + kTok < n_new) walk(j0 + kTok, nxt);
    } else {
      for (int c = warp; c < n; c += workers) {   // k . q of every token: a warp per token
        float kq = 0.f;
        for (int d = lane; d < D; d += 32) kq = fmaf(sk[c * ROW + L::at(d)], sq[c * ROW + L::at(d)], kq);
        kq = warp_sum(kq);
        if (lane == 0) skq[c * 4] = kq;
      }
      // the workers alone meet here (barrier 1): the walker warp is on its way through the next stage's gates
      asm volatile("bar.sync 1, %0;" ::"r"(wthreads) : "memory");
      for (int c = 0; c < n; ++c) {
        const float vj = valid ? sv[c * CW + j] : (is_n ? 1.f : 0.f);
        const float F = cur[c * 4 + 0], I = cur[c * 4 + 1];
        const float* qb = sq + c * ROW + ks * L::SL;
        const float* kb = sk + c * ROW + ks * L::SL;
        float2 d[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
        const float2 F2 = make_float2(F, F), w2 = make_float2(I * vj, I * vj);
#pragma unroll
        for (int r = 0; r < R; r += 4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qb + r);
          const float4 k4 = *reinterpret_cast<const float4*>(kb + r);
          d[0] = __ffma2_rn(S[r / 2], make_float2(q4.x, q4.y), d[0]);
          d[1] = __ffma2_rn(S[r / 2 + 1], make_float2(q4.z, q4.w), d[1]);
          S[r / 2] = __ffma2_rn(make_float2(k4.x, k4.y), w2, __fmul2_rn(F2, S[r / 2]));
          S[r / 2 + 1] = __ffma2_rn(make_float2(k4.z, k4.w), w2, __fmul2_rn(F2, S[r / 2 + 1]));
        }
        const float ds = slice_sum((d[0].x + d[0].y) + (d[1].x + d[1].y), KS);
        if (ks == 0) {
          const float num = fmaf(F, ds, I * skq[c * 4] * vj);
          if (valid) so[c * CW + j] = num;
          else if (is_n) sden[c] = num;
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < n * ncol; i += blockDim.x) {
      const int c = i / ncol, col = i - c * ncol;
      so[c * CW + col] *= 1.0f / (fmaxf(fabsf(sden[c]), cur[c * 4 + 2]) + 1e-6f);
    }
    __syncthreads();
    gated_unit_norm_rows<T>(a, so, part, sinv, stage, pg, h, c0, ncol, t0 + j0, n);
    __syncthreads();
  }
  if (slot != a.reserved_slot) {
    store_state<R>(S, a, slot, h, c0 + j, valid, ks);
    if (vt == 0 && is_n) {
      float* dst = nvec + ((int64_t)slot * H + h) * D;
#pragma unroll
      for (int r = 0; r < R; r += 2) {
        const int i = ks * R + r;
        if (i < D) dst[i] = S[r / 2].x;
        if (i + 1 < D) dst[i + 1] = S[r / 2].y;
      }
    }
    if (vt == 0 && walker_warp && lane == 0) mstate[(int64_t)slot * H + h] = mrun;
  }
  if (a.VT > 1) cooperative_groups::this_cluster().sync();   // nobody leaves while its sums may still be read
}

// How a (head, sequence) is laid out on CTAs and threads.
struct RecurShape {
  int R, KS, VT, CW, threads, tok;
  size_t smem(int key_rows) const {   // key_rows: staged key-sized rows per token (2 delta, 3 wkv)
    return sizeof(float) * ((size_t)key_rows * tok * KS * (R + 4) + (size_t)2 * tok * CW + tok * 4 + 4 * kTokMax);
  }
  // tokens per stage: as many as a portion has, up to kTokMax, within 96 KB of shared memory (longer stages outrun the registers that load a stage ahead: 64 tokens measured 2-4 % slower than 32 at heads of 128 x 128 and 64 x 64)
  void pick_tok(int max_new, int key_rows) {
    tok = 1;
    while (tok < kTokMax && tok < max_new) tok <<= 1;
    while (tok > 1 && smem(key_rows) > 96 * 1024) tok >>= 1;
  }
};

// VT: value columns go to 2 or 4 CTAs (a cluster) while a CTA keeps 32 columns or more and 512 threads (fewer warps
// per CTA lost more than the extra CTAs won: wkv 64 x 64, 2.28 against 2.06 ms) and the step has few (head, sequence)
// pairs for the SMs - and to as many as it takes (up to 8) for the CTA to fit 1024 threads;
// R: the shortest register slice in {8, 16, 32} whose CTA fits 512 threads (128 registers a thread), else 1024;
// KS: the power of two with KS * R >= D.  threads == 0: no layout (D or Dv too large).
// `extra`: columns every CTA keeps beside its share of the value columns (the matrix memory's normalizer column).
inline RecurShape recur_shape(int D, int Dv, int pairs, int max_new, int extra = 0) {
  RecurShape s{};
  const int forced = test_options().recur_layout.load();
  if (forced > 0) {   // tests and measurements: 100 * VT + R, taken when it fits
    s.VT = forced / 100;
    s.R = forced % 100;
    if (s.VT >= 1 && s.VT <= 8 && Dv % s.VT == 0 && (s.R == 8 || s.R == 16 || s.R == 32)) {
      s.CW = Dv / s.VT;
      s.KS = 1;
      while (s.KS * s.R < D) s.KS <<= 1;
      if (s.KS <= kMaxSlices && (s.CW + extra) * s.KS <= 1024 - 32 * extra) {
        s.threads = cdiv((s.CW + extra) * s.KS, 32) * 32;
        return s;
      }
    }
    s = RecurShape{};
  }
  if (max_new == 1) {
    // single tokens: the step is the state's trip through the registers, so many small CTAs (several per SM): columns
    // in runs of 32 where they divide so, the longest slices
    s.VT = 1;
    while (s.VT < 8 && Dv % (2 * s.VT) == 0 && Dv / (2 * s.VT) >= 32) s.VT *= 2;
    s.CW = Dv / s.VT;
    for (int r = 32; r >= 8 && s.R == 0; r >>= 1) {
      int ks = 1;
      while (ks * r < D) ks <<= 1;
      if (ks <= kMaxSlices && (s.CW + extra) * ks <= 512 + 32 * extra) s.R = r, s.KS = ks;
    }
    if (s.R != 0) {
      s.threads = cdiv((s.CW + extra) * s.KS, 32) * 32;
      return s;
    }
    s = RecurShape{};
  }
  int ks8 = 1;   // slices of 8 rows
  while (ks8 * 8 < D) ks8 <<= 1;
  s.VT = 1;
  while (s.VT < 4 && Dv % (2 * s.VT) == 0 && Dv / (2 * s.VT) >= 32 && (Dv / (2 * s.VT)) * ks8 >= 512 &&
         (int64_t)pairs * s.VT < 2 * sm_count())
    s.VT *= 2;
  for (;; s.VT *= 2) {
    s.CW = Dv / s.VT;
    s.R = 0;
    for (int limit = 512; limit <= 1024 && s.R == 0; limit *= 2)
      for (int r = 8; r <= 32 && s.R == 0; r <<= 1) {
        int ks = 1;
        while (ks * r < D) ks <<= 1;
        if (ks <= kMaxSlices && (s.CW + extra) * ks <= (limit < 1024 ? limit + 32 * extra : limit - 32 * extra)) s.R = r, s.KS = ks;
      }
    if (s.R != 0) break;
    if (s.VT >= 8 || Dv % (2 * s.VT) != 0) return s;   // threads stays 0
  }
  s.threads = cdiv((s.CW + extra) * s.KS, 32) * 32;
  return s;
}

template <typename K, typename... Args>
cudaError_t launch_clustered(K kern, dim3 grid, int threads, size_t smem, cudaStream_t st, int cluster, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = cluster > 1 ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, args...);
}

template <int R>
constexpr int max_recur_smem(int key_rows) {
  // key rows of at most kMaxKeyDim numbers: KS <= kMaxKeyDim / R slices of R + 4 floats
  (void)key_rows;
  return 200 * 1024;   // a ceiling for every shape; a launch asks for what its stage size needs (pick_tok: <= 96 KB)
}

template <typename T, int R, int MAXT>
int launch_delta(dim3 grid, const RecurShape& sh, cudaStream_t st, const float* qkv, int64_t qkv_stride,
                 const void* proj, int64_t proj_stride, int b_off, int a_off, const float* A_log, const float* dt_bias,
                 int G, const RecurArgs& a) {
  // the attribute is set once per kernel: to what the largest shape needs, not to this launch's size
  static std::atomic<uint64_t> attr{0};
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem((const void*)delta_rule_kernel<T, R, MAXT>, max_recur_smem<R>(2), attr));
  CVLLM_CHECK_CUDA(launch_clustered(delta_rule_kernel<T, R, MAXT>, grid, sh.threads, sh.smem(2), st, sh.VT, qkv,
                                    qkv_stride, static_cast<const T*>(proj), proj_stride, b_off, a_off, A_log, dt_bias,
                                    G, a));
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

template <typename T, int R, int MAXT>
int launch_wkv(dim3 grid, const RecurShape& sh, cudaStream_t st, const void* r, int64_t r_stride, const void* k,
               int64_t k_stride, const void* v, int64_t v_stride, const void* w_raw, int64_t w_stride, const float* w0,
               const float* bonus, const RecurArgs& a) {
  static std::atomic<uint64_t> attr{0};
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem((const void*)wkv_scan_kernel<T, R, MAXT>, max_recur_smem<R>(3), attr));
  CVLLM_CHECK_CUDA(launch_clustered(wkv_scan_kernel<T, R, MAXT>, grid, sh.threads, sh.smem(3), st, sh.VT,
                                    static_cast<const T*>(r), r_stride, static_cast<const T*>(k), k_stride,
                                    static_cast<const T*>(v), v_stride, static_cast<const T*>(w_raw), w_stride, w0,
                                    bonus, a));
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

template <typename T, int R, int MAXT>
int launch_general_delta(dim3 grid, const RecurShape& sh, cudaStream_t st, const void* proj, int64_t proj_stride,
                         int r_off, int k_off, int v_off, int a_off, const void* w_raw, int64_t w_stride,
                         const float* w0, float rate, const RecurArgs& a) {
  static std::atomic<uint64_t> attr{0};
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem((const void*)general_delta_kernel<T, R, MAXT>, max_recur_smem<R>(5), attr));
  CVLLM_CHECK_CUDA(launch_clustered(general_delta_kernel<T, R, MAXT>, grid, sh.threads, sh.smem(5), st, sh.VT,
                                    static_cast<const T*>(proj), proj_stride, r_off, k_off, v_off, a_off,
                                    static_cast<const T*>(w_raw), w_stride, w0, rate, a));
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

template <typename T, int R, int MAXT>
int launch_matrix_memory(dim3 grid, const RecurShape& sh, cudaStream_t st, const void* proj, int64_t proj_stride,
                         int q_off, int k_off, int v_off, int i_off, int f_off, float cap, float q_scale, float* nvec,
                         float* mstate, const RecurArgs& a) {
  static std::atomic<uint64_t> attr{0};
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem((const void*)matrix_memory_kernel<T, R, MAXT>, max_recur_smem<R>(2), attr));
  // + the warp that walks the gates; + the two stages' gate records
  CVLLM_CHECK_CUDA(launch_clustered(matrix_memory_kernel<T, R, MAXT>, grid, sh.threads + 32,
                                    sh.smem(2) + sizeof(float) * 8 * kTokMax, st, sh.VT,
                                    static_cast<const T*>(proj), proj_stride, q_off, k_off, v_off, i_off, f_off, cap,
                                    q_scale, nvec, mstate, a));
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

}  // namespace
}  // namespace cvllm

using namespace cvllm;

static int recur_dtype_ok(int dtype) { return dtype == CVLLM_BF16 || dtype == CVLLM_F32; }

extern "C" int cvllm_token_shift_mix(const void* h, int64_t h_stride, const float* mu, int S, int W, void* shift_state,
                                     const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                                     const int32_t* batch_mapping, int B, int max_new, void* out, int64_t total_tokens,
                                     int reserved_slot, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(B >= 0 && max_new >= 0 && S > 0 && W > 0);
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(h && mu && shift_state && batch_mapping && out && recur_dtype_ok(dtype));
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : (positions != nullptr && max_new == 1));
  CVLLM_CHECK_SUPPORTED(B <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  const StepGeom g{cu_seqlens_q, seq_start, positions, batch_mapping};
  const dim3 grid(cdiv(max_new, kShiftTokens), B);
  if (dtype == CVLLM_BF16) {
    token_shift_mix_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h), h_stride, mu, S, W,
                                                                static_cast<const __nv_bfloat16*>(shift_state), g,
                                                                static_cast<__nv_bfloat16*>(out), total_tokens);
    token_shift_update_kernel<__nv_bfloat16><<<B, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(h), h_stride, W,
                                                                static_cast<__nv_bfloat16*>(shift_state), g,
                                                                reserved_slot);
  } else {
    token_shift_mix_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(h), h_stride, mu, S, W,
                                                        static_cast<const float*>(shift_state), g,
                                                        static_cast<float*>(out), total_tokens);
    token_shift_update_kernel<float><<<B, 256, 0, st>>>(static_cast<const float*>(h), h_stride, W,
                                                        static_cast<float*>(shift_state), g, reserved_slot);
  }
  CVLLM_CHECK_LAUNCHES(2);
  return CVLLM_OK;
}

// R rows per slice; CTAs of up to 512 threads get twice the registers of larger ones
#define CVLLM_RECUR_BY_R(MACRO, T)                                                   \
  switch (sh.R) {                                                                    \
    case 8: return sh.threads <= 512 ? MACRO(T, 8, 512) : MACRO(T, 8, 1024);         \
    case 16: return sh.threads <= 512 ? MACRO(T, 16, 512) : MACRO(T, 16, 1024);      \
    default: return sh.threads <= 512 ? MACRO(T, 32, 512) : MACRO(T, 32, 1024);      \
  }

extern "C" int cvllm_delta_rule(const float* qkv, int64_t qkv_stride, const void* proj, int64_t proj_stride, int b_off,
                                int a_off, const float* A_log, const float* dt_bias, float* state, const void* gate,
                                int64_t gate_stride, int gate_off, const float* norm_w, int norm_head_stride, float eps,
                                const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                                const int32_t* batch_mapping, int B, int max_new, void* out, int64_t out_stride, int H,
                                int G, int D, int Dv, int reserved_slot, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(B >= 0 && max_new >= 0 && H > 0 && G > 0 && H % G == 0 && D > 0 && Dv > 0);
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(qkv && proj && A_log && dt_bias && state && gate && norm_w && batch_mapping && out &&
                  recur_dtype_ok(dtype));
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : (positions != nullptr && max_new == 1));
  CVLLM_CHECK_SUPPORTED(D <= kMaxKeyDim && Dv <= kMaxValueDim && H <= 65535 && B <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  RecurShape sh = recur_shape(D, Dv, H * B, max_new);
  sh.pick_tok(max_new, 2);
  CVLLM_CHECK_SUPPORTED(sh.threads > 0 && sh.threads <= 1024 && (int64_t)H * sh.VT <= 2147483647);
  RecurArgs a{{cu_seqlens_q, seq_start, positions, batch_mapping}, state, gate, gate_stride, gate_off, norm_w,
              norm_head_stride, eps, out, out_stride, H, D, Dv, reserved_slot, sh.KS, sh.VT, sh.CW, sh.tok};
  const dim3 grid(H * sh.VT, B);
#define CVLLM_DELTA(T, RR, MT) \
  launch_delta<T, RR, MT>(grid, sh, st, qkv, qkv_stride, proj, proj_stride, b_off, a_off, A_log, dt_bias, G, a)
  if (dtype == CVLLM_BF16) { CVLLM_RECUR_BY_R(CVLLM_DELTA, __nv_bfloat16) }
  CVLLM_RECUR_BY_R(CVLLM_DELTA, float)
#undef CVLLM_DELTA
}

extern "C" int cvllm_wkv_scan(const void* r, int64_t r_stride, const void* k, int64_t k_stride, const void* v,
                              int64_t v_stride, const void* w_raw, int64_t w_stride, const float* w0,
                              const float* bonus, float* state, const void* gate, int64_t gate_stride, int gate_off,
                              const float* norm_w, int norm_head_stride, float eps, const int32_t* cu_seqlens_q,
                              const int32_t* seq_start, const int32_t* positions, const int32_t* batch_mapping, int B,
                              int max_new, void* out, int64_t out_stride, int H, int D, int reserved_slot, int dtype,
                              cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(B >= 0 && max_new >= 0 && H > 0 && D > 0);
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(r && k && v && w_raw && w0 && bonus && state && gate && norm_w && batch_mapping && out &&
                  recur_dtype_ok(dtype));
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : (positions != nullptr && max_new == 1));
  CVLLM_CHECK_SUPPORTED(D <= kMaxValueDim && H <= 65535 && B <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  RecurShape sh = recur_shape(D, D, H * B, max_new);
  sh.pick_tok(max_new, 3);
  CVLLM_CHECK_SUPPORTED(sh.threads > 0 && sh.threads <= 1024 && (int64_t)H * sh.VT <= 2147483647);
  RecurArgs a{{cu_seqlens_q, seq_start, positions, batch_mapping}, state, gate, gate_stride, gate_off, norm_w,
              norm_head_stride, eps, out, out_stride, H, D, D, reserved_slot, sh.KS, sh.VT, sh.CW, sh.tok};
  const dim3 grid(H * sh.VT, B);
#define CVLLM_WKV(T, RR, MT) \
  launch_wkv<T, RR, MT>(grid, sh, st, r, r_stride, k, k_stride, v, v_stride, w_raw, w_stride, w0, bonus, a)
  if (dtype == CVLLM_BF16) { CVLLM_RECUR_BY_R(CVLLM_WKV, __nv_bfloat16) }
  CVLLM_RECUR_BY_R(CVLLM_WKV, float)
#undef CVLLM_WKV
}

extern "C" int cvllm_general_delta(const void* proj, int64_t proj_stride, int r_off, int k_off, int v_off, int a_off,
                                   const void* w_raw, int64_t w_stride, const float* w0, float rate, float* state,
                                   int gate_off, int gate_kind, const float* norm_w, int norm_head_stride, float eps,
                                   const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                                   const int32_t* batch_mapping, int B, int max_new, void* out, int64_t out_stride,
                                   int H, int D, int reserved_slot, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(B >= 0 && max_new >= 0 && H > 0 && D > 0);
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(proj && w_raw && w0 && state && norm_w && batch_mapping && out && recur_dtype_ok(dtype));
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : (positions != nullptr && max_new == 1));
  CVLLM_CHECK_SUPPORTED(D <= kMaxValueDim && H <= 65535 && B <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  RecurShape sh = recur_shape(D, D, H * B, max_new);
  sh.pick_tok(max_new, 5);
  CVLLM_CHECK_SUPPORTED(sh.threads > 0 && sh.threads <= 1024 && (int64_t)H * sh.VT <= 2147483647);
  RecurArgs a{{cu_seqlens_q, seq_start, positions, batch_mapping}, state, proj, proj_stride, gate_off, norm_w,
              norm_head_stride, eps, out, out_stride, H, D, D, reserved_slot, sh.KS, sh.VT, sh.CW, sh.tok, gate_kind};
  const dim3 grid(H * sh.VT, B);
#define CVLLM_GDELTA(T, RR, MT)                                                                                    \
  launch_general_delta<T, RR, MT>(grid, sh, st, proj, proj_stride, r_off, k_off, v_off, a_off, w_raw, w_stride, w0, \
                                  rate, a)
  if (dtype == CVLLM_BF16) { CVLLM_RECUR_BY_R(CVLLM_GDELTA, __nv_bfloat16) }
  CVLLM_RECUR_BY_R(CVLLM_GDELTA, float)
#undef CVLLM_GDELTA
}

extern "C" int cvllm_matrix_memory(const void* proj, int64_t proj_stride, int q_off, int k_off, int v_off, int i_off,
                                   int f_off, float cap, float q_scale, float* state, float* nvec, float* mstate,
                                   int gate_off, int gate_kind, const float* norm_w, int norm_head_stride, float eps,
                                   const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                                   const int32_t* batch_mapping, int B, int max_new, void* out, int64_t out_stride,
                                   int H, int D, int Dv, int reserved_slot, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(B >= 0 && max_new >= 0 && H > 0 && D > 0 && Dv > 0 && cap > 0.f);
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(proj && state && nvec && mstate && norm_w && batch_mapping && out && recur_dtype_ok(dtype));
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : (positions != nullptr && max_new == 1));
  CVLLM_CHECK_SUPPORTED(D <= kMaxKeyDim && Dv <= kMaxValueDim && H <= 65535 && B <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  RecurShape sh = recur_shape(D, Dv, H * B, max_new, 1);   // one more column per CTA: the normalizer
  sh.pick_tok(max_new, 2);
  CVLLM_CHECK_SUPPORTED(sh.threads > 0 && sh.threads <= 1024 && (int64_t)H * sh.VT <= 2147483647);
  RecurArgs a{{cu_seqlens_q, seq_start, positions, batch_mapping}, state, proj, proj_stride, gate_off, norm_w,
              norm_head_stride, eps, out, out_stride, H, D, Dv, reserved_slot, sh.KS, sh.VT, sh.CW, sh.tok, gate_kind};
  const dim3 grid(H * sh.VT, B);
#define CVLLM_MMEM(T, RR, MT)                                                                                       \
  launch_matrix_memory<T, RR, MT>(grid, sh, st, proj, proj_stride, q_off, k_off, v_off, i_off, f_off, cap, q_scale, \
                                  nvec, mstate, a)
  RecurShape sel = sh;      // the launch bound counts the walking warp
  sel.threads += 32;
#define CVLLM_MMEM_BY_T(T, RR) \
  return sel.threads <= 512 ? CVLLM_MMEM(T, RR, 512) : sel.threads <= 640 ? CVLLM_MMEM(T, RR, 640) : CVLLM_MMEM(T, RR, 1024)
  // CTAs of up to 640 threads (512 of columns, the normalizer's slices, the walking warp) keep 96 registers a thread
#define CVLLM_MMEM_BY_R(T)                 \
  switch (sel.R) {                         \
    case 8: CVLLM_MMEM_BY_T(T, 8);         \
    case 16: CVLLM_MMEM_BY_T(T, 16);       \
    default: CVLLM_MMEM_BY_T(T, 32);       \
  }
  if (dtype == CVLLM_BF16) { CVLLM_MMEM_BY_R(__nv_bfloat16) }
  CVLLM_MMEM_BY_R(float)
#undef CVLLM_MMEM_BY_R
#undef CVLLM_MMEM_BY_T
#undef CVLLM_MMEM
}
