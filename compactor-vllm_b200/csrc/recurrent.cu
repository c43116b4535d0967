// Linear-attention mixers whose per-head state is a [key, value] matrix carried from token to token:
//
//   gated delta rule   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//   wkv                o = (S + diag(bonus) k v^T)^T r;  S <- diag(w) S + k v^T          (w per key channel)
//
// followed, inside the same kernel, by each head's unit norm (o / sqrt(mean(o^2) + eps)), a weight and a gate:
// out = unit(o) * norm_w * silu(gate).  Also the token shift in front of the wkv projections.
//
//   cvllm_token_shift_mix   out[s, t, :] = h_t + (h_(t-1) - h_t) * mu[s, :], the slot's last row carried between steps
//   cvllm_delta_rule        unit q / k, beta, decay, the recurrence and the gated norm
//   cvllm_wkv_scan          decays from their raw logits, the recurrence and the gated norm
//
// Geometry of a step: cu_q [B + 1] token offsets and seq_start [B] first positions of the portions, batch_mapping [B]
// slots of the state pool; cu_q == NULL means one token per sequence at positions[b] (decode steps, CUDA-graph
// replays).  A portion that starts at position 0 starts from a zero state whatever the slot holds.  States, decays,
// gates of the recurrence, norms and the outputs before the final rounding are fp32.
//
// Recurrence kernels: CTA = (head, sequence); thread (j, s) keeps rows s * R .. s * R + R - 1 of column j of the state in
// registers (KS = 4 slices of the key dimension, padded to DK = 4 R rows; padded rows stay zero), so a token costs R
// multiply-adds per dot product and two shuffles to sum the slices.  Tokens are staged kTok at a time in shared
// memory (keys in the padded slice layout, read as 16-byte broadcasts); the outputs of those tokens wait there for
// the norm, which runs once per stage with a warp per token.
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
// ---------------------------------------------------------------------------------------------------------
constexpr int kTok = 16;   // tokens staged at a time
constexpr int KS = 4;      // slices of the key dimension
constexpr int kMaxValueDim = 256;

template <int R>
struct Lay {
  static constexpr int SL = R + 4;        // floats per slice in shared memory (the pad keeps 16-byte loads conflict-free)
  static constexpr int ROW = KS * SL;     // floats per staged key-sized row
  __device__ static __forceinline__ int at(int i) { return (i / R) * SL + (i % R); }
};

__device__ __forceinline__ float slice_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

struct RecurArgs {
  StepGeom g;
  float* state;            // [slots, H, D, Dv]
  const void* gate;        // [T, ..] model type: gate logits of (token, head, value channel) at gate_off + h * Dv + j
  int64_t gate_stride;
  int gate_off;
  const float* norm_w;     // weight of value channel j of head h at h * norm_head_stride + j
  int norm_head_stride;
  float eps;
  void* out;               // [T, ..] model type, head h at columns h * Dv
  int64_t out_stride;
  int H, D, Dv, reserved_slot;
};

// the outputs of `n` staged tokens (so [kTok][Dv] fp32) -> unit norm per token, weight, gate, rounded to the model type
template <typename T>
__device__ __forceinline__ void gated_unit_norm_rows(const RecurArgs& a, const float* so, int h, int tok0, int n) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const T* gate = static_cast<const T*>(a.gate);
  T* out = static_cast<T*>(a.out);
  for (int c = warp; c < n; c += warps) {
    const float* o = so + c * a.Dv;
    float ss = 0.f;
    for (int j = lane; j < a.Dv; j += 32) ss += o[j] * o[j];
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / (float)a.Dv + a.eps);
    const int64_t t = tok0 + c;
    for (int j = lane; j < a.Dv; j += 32) {
      const float gz = to_f<T>(gate[t * a.gate_stride + a.gate_off + h * a.Dv + j]);
      out[t * a.out_stride + h * a.Dv + j] = from_f<T>(o[j] * inv * a.norm_w[h * a.norm_head_stride + j] * silu_f(gz));
    }
  }
}

template <int R>
__device__ __forceinline__ void load_state(float (&S)[R], const RecurArgs& a, int slot, int h, int j, int ks, bool from_pool) {
  const float* src = a.state + ((int64_t)slot * a.H + h) * a.D * a.Dv;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = ks * R + r;
    S[r] = (from_pool && j < a.Dv && i < a.D) ? src[(int64_t)i * a.Dv + j] : 0.f;
  }
}

template <int R>
__device__ __forceinline__ void store_state(const float (&S)[R], const RecurArgs& a, int slot, int h, int j, int ks) {
  float* dst = a.state + ((int64_t)slot * a.H + h) * a.D * a.Dv;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = ks * R + r;
    if (j < a.Dv && i < a.D) dst[(int64_t)i * a.Dv + j] = S[r];
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
  const int D = a.D, Dv = a.Dv, H = a.H;
  float* sq = sm;                       // [kTok][ROW]
  float* sk = sq + kTok * L::ROW;       // [kTok][ROW]
  float* sv = sk + kTok * L::ROW;       // [kTok][Dv]
  float* so = sv + kTok * Dv;           // [kTok][Dv]
  float* sc = so + kTok * Dv;           // [kTok][4]: decay, beta, k . q
  const int h = blockIdx.x, b = blockIdx.y;
  int t0, n_new, start;
  portion(a.g, b, t0, n_new, start);
  if (n_new <= 0) return;
  const int slot = a.g.slots[b];
  const int kvh = h / (H / G);
  const int tid = threadIdx.x, j = tid / KS, ks = tid % KS;
  const int warp = tid >> 5, lane = tid & 31, warps = blockDim.x >> 5;
  for (int i = tid; i < 2 * kTok * L::ROW; i += blockDim.x) sm[i] = 0.f;   // pads and rows beyond D stay zero
  float S[R];
  load_state<R>(S, a, slot, h, j, ks, start > 0);
  const float neg_a = -expf(A_log[h]), dtb = dt_bias[h];
  const float q_scale = rsqrtf((float)D);
  const int q_col = kvh * D, k_col = G * D + kvh * D, v_col = 2 * G * D + h * Dv;
  __syncthreads();
  for (int j0 = 0; j0 < n_new; j0 += kTok) {
    const int n = min(kTok, n_new - j0);
    for (int i = tid; i < n * D; i += blockDim.x) {
      const int c = i / D, d = i - c * D;
      const float* row = qkv + (int64_t)(t0 + j0 + c) * qkv_stride;
      sq[c * L::ROW + L::at(d)] = row[q_col + d];
      sk[c * L::ROW + L::at(d)] = row[k_col + d];
    }
    for (int i = tid; i < n * Dv; i += blockDim.x) {
      const int c = i / Dv, d = i - c * Dv;
      sv[c * Dv + d] = qkv[(int64_t)(t0 + j0 + c) * qkv_stride + v_col + d];
    }
    __syncthreads();
    for (int c = warp; c < n; c += warps) {   // unit q and k, the token's scalars
      float qq = 0.f, kk = 0.f, qk = 0.f;
      for (int d = lane; d < D; d += 32) {
        const float qv = sq[c * L::ROW + L::at(d)], kv = sk[c * L::ROW + L::at(d)];
        qq += qv * qv;
        kk += kv * kv;
        qk += qv * kv;
      }
      qq = warp_sum(qq);
      kk = warp_sum(kk);
      qk = warp_sum(qk);
      const float qi = q_scale / sqrtf(qq + 1e-6f), ki = 1.0f / sqrtf(kk + 1e-6f);
      for (int d = lane; d < D; d += 32) {
        sq[c * L::ROW + L::at(d)] *= qi;
        sk[c * L::ROW + L::at(d)] *= ki;
      }
      if (lane == 0) {
        const T* pr = proj + (int64_t)(t0 + j0 + c) * proj_stride;
        sc[c * 4 + 0] = expf(neg_a * softplus_f(to_f<T>(pr[a_off + h]) + dtb));
        sc[c * 4 + 1] = sigmoid_f(to_f<T>(pr[b_off + h]));
        sc[c * 4 + 2] = qk * qi * ki;
      }
    }
    __syncthreads();
    for (int c = 0; c < n; ++c) {
      const float4* q4 = reinterpret_cast<const float4*>(sq + c * L::ROW + ks * L::SL);
      const float4* k4 = reinterpret_cast<const float4*>(sk + c * L::ROW + ks * L::SL);
      float dk = 0.f, dq = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 kq = k4[r / 4], qq = q4[r / 4];
        dk = fmaf(S[r], kq.x, dk); dq = fmaf(S[r], qq.x, dq);
        dk = fmaf(S[r + 1], kq.y, dk); dq = fmaf(S[r + 1], qq.y, dq);
        dk = fmaf(S[r + 2], kq.z, dk); dq = fmaf(S[r + 2], qq.z, dq);
        dk = fmaf(S[r + 3], kq.w, dk); dq = fmaf(S[r + 3], qq.w, dq);
      }
      dk = slice_sum(dk);
      dq = slice_sum(dq);
      const float gd = sc[c * 4 + 0], beta = sc[c * 4 + 1], kq_dot = sc[c * 4 + 2];
      const float vj = j < Dv ? sv[c * Dv + j] : 0.f;
      const float u = beta * (vj - gd * dk);
      if (ks == 0 && j < Dv) so[c * Dv + j] = fmaf(kq_dot, u, gd * dq);
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 kq = k4[r / 4];
        S[r] = fmaf(kq.x, u, gd * S[r]);
        S[r + 1] = fmaf(kq.y, u, gd * S[r + 1]);
        S[r + 2] = fmaf(kq.z, u, gd * S[r + 2]);
        S[r + 3] = fmaf(kq.w, u, gd * S[r + 3]);
      }
    }
    __syncthreads();
    gated_unit_norm_rows<T>(a, so, h, t0 + j0, n);
    __syncthreads();
  }
  if (slot != a.reserved_slot) store_state<R>(S, a, slot, h, j, ks);
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
  const int D = a.D, Dv = a.Dv, H = a.H;
  float* sr = sm;                       // [kTok][ROW]
  float* sk = sr + kTok * L::ROW;       // [kTok][ROW]
  float* sw = sk + kTok * L::ROW;       // [kTok][ROW]
  float* sv = sw + kTok * L::ROW;       // [kTok][Dv]
  float* so = sv + kTok * Dv;           // [kTok][Dv]
  const int h = blockIdx.x, b = blockIdx.y;
  int t0, n_new, start;
  portion(a.g, b, t0, n_new, start);
  if (n_new <= 0) return;
  const int slot = a.g.slots[b];
  const int tid = threadIdx.x, j = tid / KS, ks = tid % KS;
  for (int i = tid; i < 3 * kTok * L::ROW; i += blockDim.x) sm[i] = 0.f;   // pads and rows beyond D stay zero
  float S[R], U[R];
  load_state<R>(S, a, slot, h, j, ks, start > 0);
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int i = ks * R + r;
    U[r] = i < D ? bonus[h * D + i] : 0.f;
  }
  __syncthreads();
  for (int j0 = 0; j0 < n_new; j0 += kTok) {
    const int n = min(kTok, n_new - j0);
    for (int i = tid; i < n * D; i += blockDim.x) {
      const int c = i / D, d = i - c * D;
      const int64_t t = t0 + j0 + c;
      const int col = h * D + d;
      sr[c * L::ROW + L::at(d)] = to_f<T>(rp[t * r_stride + col]);
      sk[c * L::ROW + L::at(d)] = to_f<T>(kp[t * k_stride + col]);
      sw[c * L::ROW + L::at(d)] = expf(-expf(to_f<T>(wp[t * w_stride + col]) + w0[col]));
    }
    for (int i = tid; i < n * Dv; i += blockDim.x) {
      const int c = i / Dv, d = i - c * Dv;
      sv[c * Dv + d] = to_f<T>(vp[(int64_t)(t0 + j0 + c) * v_stride + h * Dv + d]);
    }
    __syncthreads();
    for (int c = 0; c < n; ++c) {
      const float4* r4 = reinterpret_cast<const float4*>(sr + c * L::ROW + ks * L::SL);
      const float4* k4 = reinterpret_cast<const float4*>(sk + c * L::ROW + ks * L::SL);
      const float4* w4 = reinterpret_cast<const float4*>(sw + c * L::ROW + ks * L::SL);
      const float vj = j < Dv ? sv[c * Dv + j] : 0.f;
      float o = 0.f;
#pragma unroll
      for (int r = 0; r < R; r += 4) {
        const float4 rr = r4[r / 4], kk = k4[r / 4], ww = w4[r / 4];
        float kv;
        kv = kk.x * vj; o = fmaf(rr.x, fmaf(U[r], kv, S[r]), o); S[r] = fmaf(ww.x, S[r], kv);
        kv = kk.y * vj; o = fmaf(rr.y, fmaf(U[r + 1], kv, S[r + 1]), o); S[r + 1] = fmaf(ww.y, S[r + 1], kv);
        kv = kk.z * vj; o = fmaf(rr.z, fmaf(U[r + 2], kv, S[r + 2]), o); S[r + 2] = fmaf(ww.z, S[r + 2], kv);
        kv = kk.w * vj; o = fmaf(rr.w, fmaf(U[r + 3], kv, S[r + 3]), o); S[r + 3] = fmaf(ww.w, S[r + 3], kv);
      }
      o = slice_sum(o);
      if (ks == 0 && j < Dv) so[c * Dv + j] = o;
    }
    __syncthreads();
    gated_unit_norm_rows<T>(a, so, h, t0 + j0, n);
    __syncthreads();
  }
  if (slot != a.reserved_slot) store_state<R>(S, a, slot, h, j, ks);
}

inline int slice_rows(int D) {   // R: rows per slice, 8 .. 64 with 4 R >= D
  int r = 8;
  while (KS * r < D) r <<= 1;
  return r;
}

template <typename T, int R, int MAXT>
int launch_delta(dim3 grid, int threads, size_t smem, cudaStream_t st, const float* qkv, int64_t qkv_stride,
                 const void* proj, int64_t proj_stride, int b_off, int a_off, const float* A_log, const float* dt_bias,
                 int G, const RecurArgs& a) {
  // the attribute is set once per kernel: to what the largest value row needs, not to this launch's size
  static std::atomic<uint64_t> attr{0};
  constexpr int kMaxSmem = (int)sizeof(float) * (2 * kTok * KS * (R + 4) + 2 * kTok * kMaxValueDim + kTok * 4);
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem((const void*)delta_rule_kernel<T, R, MAXT>, kMaxSmem, attr));
  delta_rule_kernel<T, R, MAXT><<<grid, threads, smem, st>>>(qkv, qkv_stride, static_cast<const T*>(proj), proj_stride,
                                                             b_off, a_off, A_log, dt_bias, G, a);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

template <typename T, int R, int MAXT>
int launch_wkv(dim3 grid, int threads, size_t smem, cudaStream_t st, const void* r, int64_t r_stride, const void* k,
               int64_t k_stride, const void* v, int64_t v_stride, const void* w_raw, int64_t w_stride, const float* w0,
               const float* bonus, const RecurArgs& a) {
  static std::atomic<uint64_t> attr{0};
  constexpr int kMaxSmem = (int)sizeof(float) * (3 * kTok * KS * (R + 4) + 2 * kTok * kMaxValueDim);
  CVLLM_CHECK_CUDA(ensure_max_dyn_smem((const void*)wkv_scan_kernel<T, R, MAXT>, kMaxSmem, attr));
  wkv_scan_kernel<T, R, MAXT><<<grid, threads, smem, st>>>(static_cast<const T*>(r), r_stride, static_cast<const T*>(k),
                                                           k_stride, static_cast<const T*>(v), v_stride,
                                                           static_cast<const T*>(w_raw), w_stride, w0, bonus, a);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

inline int recur_threads(int Dv) { return cdiv(Dv * KS, 32) * 32; }

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
#define CVLLM_RECUR_BY_R(MACRO, T)                                              \
  switch (R) {                                                                  \
    case 8: return threads <= 512 ? MACRO(T, 8, 512) : MACRO(T, 8, 1024);       \
    case 16: return threads <= 512 ? MACRO(T, 16, 512) : MACRO(T, 16, 1024);    \
    case 32: return threads <= 512 ? MACRO(T, 32, 512) : MACRO(T, 32, 1024);    \
    default: return threads <= 512 ? MACRO(T, 64, 512) : MACRO(T, 64, 1024);    \
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
  CVLLM_CHECK_SUPPORTED(D <= 256 && Dv <= kMaxValueDim && H <= 65535 && B <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  const int R = slice_rows(D), threads = recur_threads(Dv);
  const size_t smem = sizeof(float) * ((size_t)2 * kTok * KS * (R + 4) + (size_t)2 * kTok * Dv + kTok * 4);
  RecurArgs a{{cu_seqlens_q, seq_start, positions, batch_mapping}, state, gate, gate_stride, gate_off, norm_w,
              norm_head_stride, eps, out, out_stride, H, D, Dv, reserved_slot};
  const dim3 grid(H, B);
#define CVLLM_DELTA(T, RR, MT) \
  launch_delta<T, RR, MT>(grid, threads, smem, st, qkv, qkv_stride, proj, proj_stride, b_off, a_off, A_log, dt_bias, G, a)
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
  const int R = slice_rows(D), threads = recur_threads(D);
  const size_t smem = sizeof(float) * ((size_t)3 * kTok * KS * (R + 4) + (size_t)2 * kTok * D);
  RecurArgs a{{cu_seqlens_q, seq_start, positions, batch_mapping}, state, gate, gate_stride, gate_off, norm_w,
              norm_head_stride, eps, out, out_stride, H, D, D, reserved_slot};
  const dim3 grid(H, B);
#define CVLLM_WKV(T, RR, MT) \
  launch_wkv<T, RR, MT>(grid, threads, smem, st, r, r_stride, k, k_stride, v, v_stride, w_raw, w_stride, w0, bonus, a)
  if (dtype == CVLLM_BF16) { CVLLM_RECUR_BY_R(CVLLM_WKV, __nv_bfloat16) }
  CVLLM_RECUR_BY_R(CVLLM_WKV, float)
#undef CVLLM_WKV
}
