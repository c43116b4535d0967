// Selective state-space mixer (the scalar-decay, multi-head form): per head h with state S [P, N] (P value
// channels, N state channels; head h reads the B / C rows of group h / (heads / groups)):
//     dt_t = softplus(dt_raw_t + dt_bias_h)          S_t = exp(-exp(A_log_h) dt_t) S_(t-1) + dt_t x_t B_t^T
//     y_t  = S_t C_t + D_h x_t
// in front of it a short causal convolution per channel with silu, behind it a gate silu(z) and an RMS norm in equal
// parts.  A sequence's state - S in fp32 and the last taps - 1 inputs of the convolution - lives in a slot of a state
// pool and is carried from step to step; a step brings, per sequence, any number of new tokens (a portion of a prompt
// or one decoded token).  A portion that starts at position 0 starts from a zero state whatever the slot holds, so a
// slot needs no clearing when it is handed to another sequence.
//   cvllm_causal_conv        out = silu(bias + sum_k w[:, k] * input(t - (taps - 1 - k))), fp32 out
//   cvllm_conv_state_update  the slot's last taps - 1 inputs after the step
//   cvllm_ssm_scan           the recurrence over the step's tokens, state read and written in place
//   cvllm_gated_group_norm   out = unit_norm_per_part(y * silu(z)) * weight
// Geometry of a step: cu_q [B + 1] token offsets and seq_start [B] first positions of the portions, batch_mapping [B]
// slots; cu_q == NULL means one token per sequence at positions[b] (decode steps, CUDA-graph replays).
// Everything but the stored projections is fp32.
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

constexpr int kMaxTaps = 16;
constexpr int kConvTokens = 8;   // tokens per CTA of the convolution

// grid (token tiles, B, channel tiles), 128 threads = 128 channels.  x = columns x_off .. x_off + C of proj.
// conv_state [slots, taps - 1, C]: entry s is the input at position start - (taps - 1) + s.
// MODE 0: out = silu(bias + conv);  MODE 1: out = input + bias + conv (a convolution added to its own input, no
// activation).  TO: the output's type (fp32, or the inputs' type).
template <typename T, typename TO, int MODE>
__global__ void __launch_bounds__(128) causal_conv_kernel(const T* __restrict__ proj, int64_t p_stride, int x_off, int C,
                                                          int taps, const float* __restrict__ w,
                                                          const float* __restrict__ bias,
                                                          const T* __restrict__ conv_state, StepGeom g,
                                                          TO* __restrict__ out, int64_t o_stride) {
  const int b = blockIdx.y;
  int t0, n_new, start;
  portion(g, b, t0, n_new, start);
  const int j0 = blockIdx.x * kConvTokens;
  if (j0 >= n_new) return;
  const int ch = blockIdx.z * 128 + threadIdx.x;
  if (ch >= C) return;
  const int slot = g.slots[b];
  float wk[kMaxTaps];
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) wk[k] = k < taps ? w[(int64_t)ch * taps + k] : 0.f;
  const float bv = bias ? bias[ch] : 0.f;
  const T* st = conv_state + (int64_t)slot * (taps - 1) * C + ch;
  const int j1 = min(j0 + kConvTokens, n_new);
  for (int j = j0; j < j1; ++j) {
    float acc = bv;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
      if (k < taps) {
        const int src = j - (taps - 1 - k);
        float v = 0.f;
        if (src >= 0) v = to_f<T>(proj[(int64_t)(t0 + src) * p_stride + x_off + ch]);
        else if (start + src >= 0) v = to_f<T>(st[(int64_t)(taps - 1 + src) * C]);   // start > 0: the slot's state
        acc = fmaf(wk[k], v, acc);
        if (MODE == 1 && k == taps - 1) acc += v;
      }
    }
    out[(int64_t)(t0 + j) * o_stride + ch] = from_f<TO>(MODE == 0 ? silu_f(acc) : acc);
  }
}

// The same for a compile-time number of taps: a thread walks kConvRun tokens of its channel with the last TAPS - 1
// inputs in registers, so every input is read once.  grid (token runs, B, channel tiles), 128 threads.
constexpr int kConvRun = 32;

template <typename T, typename TO, int TAPS, int MODE>
__global__ void __launch_bounds__(128) causal_conv_run_kernel(const T* __restrict__ proj, int64_t p_stride, int x_off,
                                                              int C, const float* __restrict__ w,
                                                              const float* __restrict__ bias,
                                                              const T* __restrict__ conv_state, StepGeom g,
                                                              TO* __restrict__ out, int64_t o_stride) {
  const int b = blockIdx.y;
  int t0, n_new, start;
  portion(g, b, t0, n_new, start);
  const int j0 = blockIdx.x * kConvRun;
  if (j0 >= n_new) return;
  const int ch = blockIdx.z * 128 + threadIdx.x;
  if (ch >= C) return;
  const int slot = g.slots[b];
  float wk[TAPS], win[TAPS];          // win[k] = input at j - (TAPS - 1 - k); win[TAPS - 1] is the current token's
#pragma unroll
  for (int k = 0; k < TAPS; ++k) wk[k] = w[(int64_t)ch * TAPS + k];
  const float bv = bias ? bias[ch] : 0.f;
  const T* st = conv_state + (int64_t)slot * (TAPS - 1) * C + ch;
  const T* in = proj + (int64_t)t0 * p_stride + x_off + ch;
#pragma unroll
  for (int k = 0; k < TAPS - 1; ++k) {
    const int src = j0 - (TAPS - 1 - k);
    float v = 0.f;
    if (src >= 0) v = to_f<T>(in[(int64_t)src * p_stride]);
    else if (start + src >= 0) v = to_f<T>(st[(int64_t)(TAPS - 1 + src) * C]);
    win[k] = v;
  }
  const int j1 = min(j0 + kConvRun, n_new);
  for (int j = j0; j < j1; ++j) {
    win[TAPS - 1] = to_f<T>(in[(int64_t)j * p_stride]);
    float acc = bv;
#pragma unroll
    for (int k = 0; k < TAPS; ++k) acc = fmaf(wk[k], win[k], acc);
    if (MODE == 1) acc += win[TAPS - 1];
    out[(int64_t)(t0 + j) * o_stride + ch] = from_f<TO>(MODE == 0 ? silu_f(acc) : acc);
#pragma unroll
    for (int k = 0; k < TAPS - 1; ++k) win[k] = win[k + 1];
  }
}

// grid (B, channel tiles), 128 threads: a thread reads what it needs of its channel's old state, then writes the new.
template <typename T>
__global__ void __launch_bounds__(128) conv_state_update_kernel(const T* __restrict__ proj, int64_t p_stride,
                                                                int x_off, int C, int taps,
                                                                T* __restrict__ conv_state, StepGeom g,
                                                                int reserved_slot) {
  const int b = blockIdx.x;
  const int ch = blockIdx.y * 128 + threadIdx.x;
  if (ch >= C) return;
  int t0, n_new, start;
  portion(g, b, t0, n_new, start);
  const int slot = g.slots[b];
  if (slot == reserved_slot || n_new <= 0) return;
  T* st = conv_state + (int64_t)slot * (taps - 1) * C + ch;
  T keep[kMaxTaps];
#pragma unroll
  for (int s = 0; s < kMaxTaps - 1; ++s) {
    if (s < taps - 1) {
      const int j = n_new - (taps - 1) + s;   // index among the new tokens of the input that entry s will hold
      if (j >= 0) keep[s] = proj[(int64_t)(t0 + j) * p_stride + x_off + ch];
      else if (start + j >= 0) keep[s] = st[(int64_t)(s + n_new) * C];
      else keep[s] = from_f<T>(0.f);
    }
  }
#pragma unroll
  for (int s = 0; s < kMaxTaps - 1; ++s)
    if (s < taps - 1) st[(int64_t)s * C] = keep[s];
}

constexpr int kScanTokens = 16;   // tokens staged per pass

template <int V>
struct IntC { static constexpr int value = V; };
constexpr int kPad = 4;           // floats between the 16-value slices of a staged B / C row (keeps 16-byte alignment)

__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(addr), "l"(gmem) : "memory");
}

__device__ __forceinline__ void cp_async16(float* smem, const float* gmem) {
  const uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(addr), "l"(gmem) : "memory");
}

// grid (heads, B * nseg, value tiles), PT * NS threads: NS slices of the state dimension (a power of two, NS * 16 >= N)
// times PT value channels; thread (pl, s) keeps S[p, 16 s .. 16 s + 15] for its TWO value channels p = p0 + pl and
// p0 + pl + PT in registers over its tokens, so that the 32 values of B_t and C_t it reads from shared memory per token
// (eight 16-byte loads) serve 64 state updates.
// xbc [T, inner + 2 G N] fp32 = conv output (x | B | C); dt_raw = column dt_off + h of proj.
// A portion is cut into nseg segments of seg tokens (nseg 1: the whole portion).  mode 0: the CTA runs the whole
// portion from the pool's state.  Long portions of steps with few CTAs run in three launches so that the segments of one
// sequence run side by side: mode 1 runs every segment but a sequence's last from a ZERO state, without output, and
// leaves the segment's end state and its summed step sizes in seg_state / seg_dt; ssm_seg_combine_kernel turns those
// into each segment's true initial state (S_init[k + 1] = exp(-a sum_dt[k]) S_init[k] + S_local[k], the recurrence
// being linear in S); mode 2 reruns every segment from its initial state with output, and a sequence's last segment
// writes the pool.
template <typename T, int NPT, bool WITH_Y>
__global__ void __launch_bounds__(256) ssm_scan_kernel(const float* __restrict__ xbc, int64_t x_stride,
                                                       const T* __restrict__ proj, int64_t p_stride, int dt_off,
                                                       const float* __restrict__ dt_bias,
                                                       const float* __restrict__ A_log, const float* __restrict__ Dp,
                                                       float* __restrict__ state, StepGeom g, float* __restrict__ y,
                                                       int64_t y_stride, int heads, int groups, int P, int N, int NS,
                                                       int PT, int reserved_slot, int mode, int nseg, int seg,
                                                       float* __restrict__ seg_state, float* __restrict__ seg_dt) {
  extern __shared__ __align__(16) float sm[];
  const int nthr = blockDim.x;
  const int PW = 2 * PT;                        // value channels per CTA
  const int NL = NS * (NPT + kPad);            // staged row of B / C: slice s starts at s * 20
  const int stage_floats = kScanTokens * (2 * NL + PW);
  float* stages = sm;                           // two stages of [B rows | C rows | x rows] for kScanTokens tokens
  float* ys = sm + 2 * stage_floats;            // [kScanTokens][PW]
  float* dts = ys + kScanTokens * PW;           // [kScanTokens]
  float* dAs = dts + kScanTokens;               // [kScanTokens]
  const int h = blockIdx.x, b = blockIdx.y / nseg, k = blockIdx.y - b * nseg, p0 = blockIdx.z * PW;
  int t0, n_new, start;
  portion(g, b, t0, n_new, start);
  const int j_begin = mode == 0 ? 0 : k * seg;
  const int j_end = mode == 0 ? n_new : min(n_new, j_begin + seg);
  if (j_begin >= j_end) return;
  const bool last_seg = j_end == n_new;
  if (mode == 1 && last_seg) return;            // nobody needs the end state of a sequence's last segment early
  const int slot = g.slots[b];
  const int tid = threadIdx.x, s = tid & (NS - 1), pl = tid / NS;
  const int inner = heads * P, grp = h / (heads / groups);
  if (slot == reserved_slot) {
    if (mode == 1) return;
    for (int i = tid; i < (j_end - j_begin) * PW; i += nthr) {
      const int j = i / PW, c = i - j * PW;
      if (p0 + c < P) y[(int64_t)(t0 + j_begin + j) * y_stride + h * P + p0 + c] = 0.f;
    }
    return;
  }
  // the padding of the staged rows and the channels past P are zero for good: the copies below never touch them
  for (int i = tid; i < 2 * stage_floats; i += nthr) stages[i] = 0.f;
  __syncthreads();
  int ns_shift = 0;
  while ((1 << ns_shift) < NS) ++ns_shift;
  // B / C rows in 16-byte pieces when every piece is aligned in global memory
  const bool vec_in = (N & 3) == 0 && (x_stride & 3) == 0 && (inner & 3) == 0 &&
                      (reinterpret_cast<uintptr_t>(xbc) & 15) == 0;
  // a chunk's inputs are copied global -> shared asynchronously, one chunk ahead of the arithmetic
  auto issue = [&](int stage, int c0) {
    const int nt = min(kScanTokens, j_end - c0);
    float* Bs = stages + stage * stage_floats;
    float* Cs = Bs + kScanTokens * NL;
    float* xs = Cs + kScanTokens * NL;
    if (vec_in) {      // 16-byte pieces: rows of NS * NPT / 4 pieces (a power of two)
      const int row_shift = ns_shift + (NPT == 16 ? 2 : 1);
      for (int i = tid; i < (nt << row_shift); i += nthr) {
        const int j = i >> row_shift, n = (i & ((1 << row_shift) - 1)) * 4;
        if (n < N) {
          const float* row = xbc + (int64_t)(t0 + c0 + j) * x_stride + inner + grp * N;
          const int at = j * NL + (n / NPT) * (NPT + kPad) + (n % NPT);
          cp_async16(Bs + at, row + n);
          cp_async16(Cs + at, row + (int64_t)groups * N + n);
        }
      }
    } else {
      const int row_shift = ns_shift + (NPT == 16 ? 4 : 3);
      for (int i = tid; i < (nt << row_shift); i += nthr) {
        const int j = i >> row_shift, n = i & ((1 << row_shift) - 1);
        if (n < N) {
          const float* row = xbc + (int64_t)(t0 + c0 + j) * x_stride + inner + grp * N;
          const int at = j * NL + (n / NPT) * (NPT + kPad) + (n % NPT);
          cp_async4(Bs + at, row + n);
          cp_async4(Cs + at, row + (int64_t)groups * N + n);
        }
      }
    }
    for (int i = tid; i < nt * PW; i += nthr) {
      const int j = i / PW, c = i - j * PW;
      if (p0 + c < P) cp_async4(xs + i, xbc + (int64_t)(t0 + c0 + j) * x_stride + h * P + p0 + c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const bool vec = (N & 3) == 0;                // 16-byte state rows
  float2 S[2][NPT / 2];          // pairs of neighbouring state channels: the arithmetic below is packed fp32x2
  float* pool_row[2];
  float* seg_row[2];
  const float* init[2];
  bool live[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int p = p0 + pl + u * PT;
    live[u] = p < P;
    pool_row[u] = state + (((int64_t)slot * heads + h) * P + p) * N + s * NPT;
    seg_row[u] = seg_state ? seg_state + ((((int64_t)b * nseg + k) * heads + h) * P + p) * N + s * NPT : nullptr;
    init[u] = mode == 2 ? seg_row[u] : ((mode == 0 && start > 0) ? pool_row[u] : nullptr);
  }
  issue(0, j_begin);
  float dt_next = (tid < min(kScanTokens, j_end - j_begin))
                      ? to_f<T>(proj[(int64_t)(t0 + j_begin + tid) * p_stride + dt_off + h]) : 0.f;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    if (init[u] && live[u] && vec) {
#pragma unroll
      for (int i = 0; i < NPT; i += 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (s * NPT + i < N) v = *reinterpret_cast<const float4*>(init[u] + i);
        S[u][i / 2] = make_float2(v.x, v.y);
        S[u][i / 2 + 1] = make_float2(v.z, v.w);
      }
    } else {
#pragma unroll
      for (int i = 0; i < NPT; i += 2) {
        const bool ok = init[u] && live[u];
        S[u][i / 2] = make_float2((ok && s * NPT + i < N) ? init[u][i] : 0.f,
                                  (ok && s * NPT + i + 1 < N) ? init[u][i + 1] : 0.f);
      }
    }
  }
  const float a = expf(A_log[h]), dsk = Dp[h], bias = dt_bias[h];
  float dt_sum = 0.f;
  int stage = 0;
  for (int c0 = j_begin; c0 < j_end; c0 += kScanTokens, stage ^= 1) {
    const int nt = min(kScanTokens, j_end - c0);
    const int c1 = c0 + kScanTokens;
    if (tid < nt) {               // step sizes of this chunk from the value fetched a chunk ago; fetch the next
      const float dt = softplus_f(dt_next + bias);
      dts[tid] = dt;
      dAs[tid] = expf(-a * dt);
    }
    if (c1 < j_end) {
      issue(stage ^ 1, c1);       // its stage was last read before the barrier that ended the previous pass
      if (tid < min(kScanTokens, j_end - c1)) dt_next = to_f<T>(proj[(int64_t)(t0 + c1 + tid) * p_stride + dt_off + h]);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();              // every thread's copies of this chunk have landed; dts / dAs are written
    const float* Bs = stages + stage * stage_floats;
    const float* Cs = Bs + kScanTokens * NL;
    const float* xs = Cs + kScanTokens * NL;
    // Tokens go in groups of four: the loads and the arithmetic of a group carry no store between them, so the four
    // tokens' shared-memory loads, FMA chains and cross-lane sums overlap; only S links one token to the next.
    auto run_group = [&](auto width, int j0) {
      constexpr int kGroup = decltype(width)::value;
      float r0[kGroup], r1[kGroup], xa[kGroup], xb[kGroup];
#pragma unroll
      for (int u = 0; u < kGroup; ++u) {
        const int j = j0 + u;
        const float dA = dAs[j], dt = dts[j];
        const float x0 = xs[j * PW + pl], x1 = xs[j * PW + pl + PT];
        const float dx0 = dt * x0, dx1 = dt * x1;
        xa[u] = x0;
        xb[u] = x1;
        dt_sum += dt;
        const float4* B4 = reinterpret_cast<const float4*>(Bs + j * NL + s * (NPT + kPad));
        const float4* C4 = reinterpret_cast<const float4*>(Cs + j * NL + s * (NPT + kPad));
        // per pair of state channels: S = dA S + (dt x) B  (a product rounded, then one FMA) and y += S C, as fp32x2
        const float2 dA2 = make_float2(dA, dA), dxa = make_float2(dx0, dx0), dxb = make_float2(dx1, dx1);
        float2 a0 = make_float2(0.f, 0.f), a1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int q = 0; q < NPT / 4; ++q) {
          const float4 bv = B4[q];
          const float2 b01 = make_float2(bv.x, bv.y), b23 = make_float2(bv.z, bv.w);
          S[0][2 * q] = __ffma2_rn(dA2, S[0][2 * q], __fmul2_rn(dxa, b01));
          S[0][2 * q + 1] = __ffma2_rn(dA2, S[0][2 * q + 1], __fmul2_rn(dxa, b23));
          S[1][2 * q] = __ffma2_rn(dA2, S[1][2 * q], __fmul2_rn(dxb, b01));
          S[1][2 * q + 1] = __ffma2_rn(dA2, S[1][2 * q + 1], __fmul2_rn(dxb, b23));
          if constexpr (WITH_Y) {
            const float4 cv = C4[q];
            const float2 c01 = make_float2(cv.x, cv.y), c23 = make_float2(cv.z, cv.w);
            a0 = __ffma2_rn(S[0][2 * q], c01, a0);
            a0 = __ffma2_rn(S[0][2 * q + 1], c23, a0);
            a1 = __ffma2_rn(S[1][2 * q], c01, a1);
            a1 = __ffma2_rn(S[1][2 * q + 1], c23, a1);
          }
        }
        r0[u] = a0.x + a0.y;
        r1[u] = a1.x + a1.y;
      }
      if constexpr (WITH_Y) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {     // NS is the same for every thread: no divergence
          if (o < NS) {
#pragma unroll
            for (int u = 0; u < kGroup; ++u) {
              r0[u] += __shfl_xor_sync(0xffffffffu, r0[u], o);
              r1[u] += __shfl_xor_sync(0xffffffffu, r1[u], o);
            }
          }
        }
        if (s == 0) {
#pragma unroll
          for (int u = 0; u < kGroup; ++u) {
            ys[(j0 + u) * PW + pl] = r0[u] + dsk * xa[u];
            ys[(j0 + u) * PW + pl + PT] = r1[u] + dsk * xb[u];
          }
        }
      }
    };
    int j0 = 0;
    for (; j0 + 4 <= nt; j0 += 4) run_group(IntC<4>{}, j0);
    for (; j0 < nt; ++j0) run_group(IntC<1>{}, j0);       // a chunk's last tokens, and single-token steps
    __syncthreads();              // ys complete; this chunk's stage and dts may be overwritten from here on
    if (mode == 1) continue;
    for (int i = tid; i < nt * PW; i += nthr) {
      const int j = i / PW, c = i - j * PW;
      if (p0 + c < P) y[(int64_t)(t0 + c0 + j) * y_stride + h * P + p0 + c] = ys[i];
    }
  }
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    float* dst = mode == 1 ? seg_row[u] : ((mode == 0 || last_seg) ? pool_row[u] : nullptr);
    if (!dst || !live[u]) continue;
    if (vec) {
#pragma unroll
      for (int i = 0; i < NPT; i += 4)
        if (s * NPT + i < N)
          *reinterpret_cast<float4*>(dst + i) =
              make_float4(S[u][i / 2].x, S[u][i / 2].y, S[u][i / 2 + 1].x, S[u][i / 2 + 1].y);
    } else {
#pragma unroll
      for (int i = 0; i < NPT; i += 2) {
        if (s * NPT + i < N) dst[i] = S[u][i / 2].x;
        if (s * NPT + i + 1 < N) dst[i + 1] = S[u][i / 2].y;
      }
    }
  }
  if (mode == 1 && tid == 0 && blockIdx.z == 0) seg_dt[((int64_t)b * nseg + k) * heads + h] = dt_sum;
}

// grid (heads, B), 256 threads over the P * N state entries of a head: seg_state[b, k] (the segment's local end state,
// from a zero start) becomes the segment's initial state, k = 0 .. the sequence's segment count - 1.
__global__ void __launch_bounds__(256) ssm_seg_combine_kernel(float* __restrict__ seg_state,
                                                              const float* __restrict__ seg_dt,
                                                              const float* __restrict__ state,
                                                              const float* __restrict__ A_log, StepGeom g, int heads,
                                                              int P, int N, int nseg, int seg, int reserved_slot) {
  const int h = blockIdx.x, b = blockIdx.y;
  int t0, n_new, start;
  portion(g, b, t0, n_new, start);
  const int slot = g.slots[b];
  if (slot == reserved_slot || n_new <= 0) return;
  const int mine = (n_new + seg - 1) / seg;
  const float a = expf(A_log[h]);
  const int64_t per = (int64_t)P * N;
  for (int e = threadIdx.x; e < per; e += 256) {
    float cur = start > 0 ? state[((int64_t)slot * heads + h) * per + e] : 0.f;
    for (int k = 0; k < mine; ++k) {
      float* cell = seg_state + (((int64_t)b * nseg + k) * heads + h) * per + e;
      const float local = k < mine - 1 ? *cell : 0.f;
      *cell = cur;
      if (k < mine - 1) cur = fmaf(expf(-a * seg_dt[((int64_t)b * nseg + k) * heads + h]), cur, local);
    }
  }
}

// grid (T, parts), 128 threads.  out[t, c] = v / sqrt(mean_part(v^2) + eps) * w[c], v = y[t, c] * silu(z[t, c]).
template <typename T>
__global__ void __launch_bounds__(128) gated_group_norm_kernel(const float* __restrict__ y, int64_t y_stride,
                                                               const T* __restrict__ z, int64_t z_stride,
                                                               const float* __restrict__ w, float eps,
                                                               T* __restrict__ out, int64_t o_stride, int part) {
  extern __shared__ float vals[];
  __shared__ float red[4];
  const int64_t t = blockIdx.x;
  const int c0 = blockIdx.y * part;
  float ss = 0.f;
  for (int i = threadIdx.x; i < part; i += 128) {
    const float v = y[t * y_stride + c0 + i] * silu_f(to_f<T>(z[t * z_stride + c0 + i]));
    vals[i] = v;
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)part + eps);
  for (int i = threadIdx.x; i < part; i += 128) out[t * o_stride + c0 + i] = from_f<T>(vals[i] * inv * w[c0 + i]);
}

// Selective scan with a decay per (channel, state channel) and a step size per channel:
//     dt_t[c] = softplus(dt_raw_t[c] + dt_bias[c])      S_t[c, n] = exp(dt_t[c] A[c, n]) S_(t-1)[c, n] + dt_t[c] x_t[c] B_t[n]
//     y_t[c]  = sum_n S_t[c, n] C_t[n] + D[c] x_t[c]     out_t[c] = y_t[c] silu(z_t[c])
// with A = -exp(A_log) [channels, N].  grid (channel tiles, B), CT * NS threads: thread (pl, s) keeps the NPT state
// channels s * NPT .. of channel c0 + pl in registers over the portion's tokens (NS a power of two, NS * NPT >= N);
// a token's B and C rows, and the tile's step sizes and inputs, are staged kSelTokens tokens at a time.  The work has
// channels * N independent recurrences and nothing else to run side by side, so NPT is chosen by the host as small as
// it takes to fill the SMs with threads (one state channel per thread for a single portion of a few thousand channels);
// the sum over n is NS lanes' shuffles.  x, dt_raw, the B | C columns and z are stored projections (model type); the
// rest is fp32.
constexpr int kSelTokens = 32;

template <typename T, int NPT>
__global__ void __launch_bounds__(256) selective_scan_kernel(const T* __restrict__ x, int64_t x_stride,
                                                             const T* __restrict__ dt_raw, int64_t dt_stride,
                                                             const float* __restrict__ dt_bias,
                                                             const T* __restrict__ bc, int64_t bc_stride, int b_off,
                                                             int c_off, const float* __restrict__ A_log,
                                                             const float* __restrict__ Dp, const T* __restrict__ z,
                                                             int64_t z_stride, int z_off, float* __restrict__ state,
                                                             StepGeom g, T* __restrict__ out, int64_t o_stride,
                                                             int inner, int N, int NS, int CT, int reserved_slot) {
  extern __shared__ __align__(16) float sm[];
  const int NSP = NS * NPT;
  float* sB = sm;                              // [kSelTokens][NSP]
  float* sC = sB + kSelTokens * NSP;           // [kSelTokens][NSP]
  float* sdt = sC + kSelTokens * NSP;          // [kSelTokens][CT]
  float* sx = sdt + kSelTokens * CT;           // [kSelTokens][CT]
  float* sy = sx + kSelTokens * CT;            // [kSelTokens][CT]
  const int b = blockIdx.y, c0 = blockIdx.x * CT;
  int t0, n_new, start;
  portion(g, b, t0, n_new, start);
  if (n_new <= 0) return;
  const int slot = g.slots[b];
  const int tid = threadIdx.x, nthr = blockDim.x, s = tid & (NS - 1), pl = tid / NS;
  const int ch = c0 + pl;
  const bool live = ch < inner;
  if (slot == reserved_slot) {
    for (int i = tid; i < n_new * CT; i += nthr) {
      const int j = i / CT, c = i - j * CT;
      if (c0 + c < inner) out[(int64_t)(t0 + j) * o_stride + c0 + c] = from_f<T>(0.f);
    }
    return;
  }
  float S[NPT], A[NPT];
  float* srow = state + ((int64_t)slot * inner + ch) * N + s * NPT;
#pragma unroll
  for (int e = 0; e < NPT; ++e) {
    const bool in = live && s * NPT + e < N;
    A[e] = in ? -expf(A_log[(int64_t)ch * N + s * NPT + e]) : 0.f;
    S[e] = (in && start > 0) ? srow[e] : 0.f;
  }
  const float dsk = live ? Dp[ch] : 0.f;
  for (int j0 = 0; j0 < n_new; j0 += kSelTokens) {
    const int n = min(kSelTokens, n_new - j0);
    for (int i = tid; i < n * NSP; i += nthr) {
      const int j = i / NSP, nn = i - j * NSP;
      const T* row = bc + (int64_t)(t0 + j0 + j) * bc_stride;
      sB[i] = nn < N ? to_f<T>(row[b_off + nn]) : 0.f;
      sC[i] = nn < N ? to_f<T>(row[c_off + nn]) : 0.f;
    }
    for (int i = tid; i < n * CT; i += nthr) {
      const int j = i / CT, c = i - j * CT;
      const bool in = c0 + c < inner;
      const int64_t t = t0 + j0 + j;
      sdt[i] = in ? softplus_f(to_f<T>(dt_raw[t * dt_stride + c0 + c]) + dt_bias[c0 + c]) : 0.f;
      sx[i] = in ? to_f<T>(x[t * x_stride + c0 + c]) : 0.f;
    }
    __syncthreads();
    for (int j = 0; j < n; ++j) {
      const float dt = sdt[j * CT + pl], xv = sx[j * CT + pl];
      const float dx = dt * xv;
      const float* Bj = sB + j * NSP + s * NPT;
      const float* Cj = sC + j * NSP + s * NPT;
      float acc = 0.f;
#pragma unroll
      for (int e = 0; e < NPT; ++e) {
        S[e] = fmaf(exp_1ulp(dt * A[e]), S[e], dx * Bj[e]);
        acc = fmaf(S[e], Cj[e], acc);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
        if (o < NS) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (s == 0) sy[j * CT + pl] = fmaf(dsk, xv, acc);
    }
    __syncthreads();
    for (int i = tid; i < n * CT; i += nthr) {
      const int j = i / CT, c = i - j * CT;
      if (c0 + c < inner) {
        const int64_t t = t0 + j0 + j;
        out[t * o_stride + c0 + c] = from_f<T>(sy[i] * silu_f(to_f<T>(z[t * z_stride + z_off + c0 + c])));
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int e = 0; e < NPT; ++e)
    if (live && s * NPT + e < N) srow[e] = S[e];
}

// state channels per thread: 8 (twice the threads, for the latencies of a sequential recurrence) up to N = 256, else 16
int scan_npt(int N) { return N <= 256 ? 8 : 16; }

int scan_slices(int N) {
  const int npt = scan_npt(N);
  int ns = 1;
  while (ns * npt < N) ns <<= 1;
  return ns;
}

// value channels per thread row: 256 / NS, but no more than half the head's channels need (a thread owns two)
int scan_rows(int NS, int P) {
  int pt = 256 / NS;
  const int need = cdiv(cdiv(P, 2) * NS, 32) * 32 / NS;   // whole warps
  return need < pt ? (need > 0 ? need : 1) : pt;
}

// Tokens per segment of a step whose longest portion has max_new tokens; 0 = portions run whole, in one launch.
// Segments cost 1.6x the instructions of the single pass, and with every SM busy the kernel is bound by instruction
// issue: they pay only when whole portions would leave at least half of the SMs idle (measured at 64-channel heads,
// state 128, 4096 tokens: 16 heads 0.98 -> 0.38 ms, 32 heads 1.04 -> 0.67 ms, 64 heads 1.09 -> 1.18-1.42 ms,
// 128 heads 1.46 -> 2.2-2.8 ms).  The length aims at three CTAs per SM, is at least 128 tokens and a multiple of the
// staging pass; the test option "ssm_segment" forces a length whatever the CTA count.
int scan_segment(int max_new, int B, int heads, int P, int N) {
  int seg = test_options().ssm_segment.load();
  if (seg <= 0) {
    const int NS = scan_slices(N);
    const int64_t ctas = (int64_t)B * heads * cdiv(P, 2 * scan_rows(NS, P));
    if (2 * ctas > (int64_t)sm_count()) return 0;
    const int want = (int)((3 * (int64_t)sm_count() + ctas - 1) / ctas);   // segments per portion
    seg = cdiv(max_new, want);
    if (seg < 128) seg = 128;
  }
  seg = cdiv(seg, kScanTokens) * kScanTokens;
  return max_new > seg ? seg : 0;
}

}  // namespace
}  // namespace cvllm

using namespace cvllm;

static int ssm_dtype_ok(int dtype) { return dtype == CVLLM_BF16 || dtype == CVLLM_F32; }

namespace {

template <typename T, typename TO, int MODE>
int launch_conv(const void* proj, int64_t proj_stride, int x_off, int channels, int taps, const float* weight,
                const float* bias, const void* conv_state, const StepGeom& g, int B, int max_new, void* out,
                int64_t out_stride, cudaStream_t st) {
  const T* in = static_cast<const T*>(proj);
  const T* cs = static_cast<const T*>(conv_state);
  TO* o = static_cast<TO*>(out);
  if (taps >= 2 && taps <= 4) {
    const dim3 rgrid(cdiv(max_new, kConvRun), B, cdiv(channels, 128));
    if (taps == 2)
      causal_conv_run_kernel<T, TO, 2, MODE><<<rgrid, 128, 0, st>>>(in, proj_stride, x_off, channels, weight, bias, cs, g, o, out_stride);
    else if (taps == 3)
      causal_conv_run_kernel<T, TO, 3, MODE><<<rgrid, 128, 0, st>>>(in, proj_stride, x_off, channels, weight, bias, cs, g, o, out_stride);
    else
      causal_conv_run_kernel<T, TO, 4, MODE><<<rgrid, 128, 0, st>>>(in, proj_stride, x_off, channels, weight, bias, cs, g, o, out_stride);
  } else {
    const dim3 grid(cdiv(max_new, kConvTokens), B, cdiv(channels, 128));
    causal_conv_kernel<T, TO, MODE><<<grid, 128, 0, st>>>(in, proj_stride, x_off, channels, taps, weight, bias, cs, g, o, out_stride);
  }
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

}  // namespace

extern "C" int cvllm_causal_conv(const void* proj, int64_t proj_stride, int x_off, int channels, int taps,
                                 const float* weight, const float* bias, const void* conv_state,
                                 const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                                 const int32_t* batch_mapping, int B, int max_new, float* out, int64_t out_stride,
                                 int dtype, cvllm_stream_t stream) {
  return cvllm_causal_conv_mode(proj, proj_stride, x_off, channels, taps, weight, bias, conv_state, cu_seqlens_q,
                                seq_start, positions, batch_mapping, B, max_new, out, out_stride, CVLLM_F32, 0, dtype,
                                stream);
}

extern "C" int cvllm_causal_conv_mode(const void* proj, int64_t proj_stride, int x_off, int channels, int taps,
                                      const float* weight, const float* bias, const void* conv_state,
                                      const int32_t* cu_seqlens_q, const int32_t* seq_start,
                                      const int32_t* positions, const int32_t* batch_mapping, int B, int max_new,
                                      void* out, int64_t out_stride, int out_dtype, int mode, int dtype,
                                      cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(B >= 0 && max_new >= 0 && channels > 0 && taps >= 1 && (mode == 0 || mode == 1));
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(proj && weight && out && batch_mapping && ssm_dtype_ok(dtype) && (taps == 1 || conv_state));
  CVLLM_CHECK_ARG(out_dtype == CVLLM_F32 || out_dtype == dtype);
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : (positions != nullptr && max_new == 1));
  CVLLM_CHECK_SUPPORTED(taps <= kMaxTaps && B <= 65535 && cdiv(channels, 128) <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  const StepGeom g{cu_seqlens_q, seq_start, positions, batch_mapping};
#define CVLLM_CONV(T, TO, MODE) \
  return launch_conv<T, TO, MODE>(proj, proj_stride, x_off, channels, taps, weight, bias, conv_state, g, B, max_new, out, out_stride, st)
  if (dtype == CVLLM_BF16) {
    if (out_dtype == CVLLM_F32) { if (mode == 0) CVLLM_CONV(__nv_bfloat16, float, 0); CVLLM_CONV(__nv_bfloat16, float, 1); }
    if (mode == 0) CVLLM_CONV(__nv_bfloat16, __nv_bfloat16, 0);
    CVLLM_CONV(__nv_bfloat16, __nv_bfloat16, 1);
  }
  if (mode == 0) CVLLM_CONV(float, float, 0);
  CVLLM_CONV(float, float, 1);
#undef CVLLM_CONV
}

extern "C" int cvllm_conv_state_update(const void* proj, int64_t proj_stride, int x_off, int channels, int taps,
                                       void* conv_state, const int32_t* cu_seqlens_q, const int32_t* seq_start,
                                       const int32_t* positions, const int32_t* batch_mapping, int B,
                                       int reserved_slot, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(B >= 0 && channels > 0 && taps >= 1);
  if (B == 0 || taps == 1) return CVLLM_OK;
  CVLLM_CHECK_ARG(proj && conv_state && batch_mapping && ssm_dtype_ok(dtype));
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : positions != nullptr);
  CVLLM_CHECK_SUPPORTED(taps <= kMaxTaps && cdiv(channels, 128) <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  const StepGeom g{cu_seqlens_q, seq_start, positions, batch_mapping};
  const dim3 grid(B, cdiv(channels, 128));
  if (dtype == CVLLM_BF16)
    conv_state_update_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(static_cast<const __nv_bfloat16*>(proj), proj_stride,
                                                                  x_off, channels, taps,
                                                                  static_cast<__nv_bfloat16*>(conv_state), g,
                                                                  reserved_slot);
  else
    conv_state_update_kernel<float><<<grid, 128, 0, st>>>(static_cast<const float*>(proj), proj_stride, x_off, channels,
                                                          taps, static_cast<float*>(conv_state), g, reserved_slot);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" size_t cvllm_ssm_scan_workspace_bytes(int B, int max_new, int heads, int P, int N) {
  const int seg = scan_segment(max_new, B, heads, P, N);
  if (seg <= 0) return 0;
  const size_t nseg = (size_t)cdiv(max_new, seg);
  return sizeof(float) * (size_t)B * nseg * heads * ((size_t)P * N + 1);
}

extern "C" int cvllm_ssm_scan(const float* xbc, int64_t xbc_stride, const void* proj, int64_t proj_stride, int dt_off,
                              const float* dt_bias, const float* A_log, const float* D, float* state,
                              const int32_t* cu_seqlens_q, const int32_t* seq_start, const int32_t* positions,
                              const int32_t* batch_mapping, int B, int max_new, float* y, int64_t y_stride, int heads,
                              int groups, int P, int N, int reserved_slot, float* workspace, size_t workspace_bytes,
                              int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(B >= 0 && heads > 0 && groups > 0 && heads % groups == 0 && P > 0 && N > 0 && max_new >= 0);
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(xbc && proj && dt_bias && A_log && D && state && batch_mapping && y && ssm_dtype_ok(dtype));
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : (positions != nullptr && max_new == 1));
  const int NS = scan_slices(N);
  CVLLM_CHECK_SUPPORTED(NS <= 32);
  const int PT = scan_rows(NS, P);
  auto st = static_cast<cudaStream_t>(stream);
  const StepGeom g{cu_seqlens_q, seq_start, positions, batch_mapping};
  const int seg = scan_segment(max_new, B, heads, P, N);
  const int nseg = seg > 0 ? cdiv(max_new, seg) : 1;
  CVLLM_CHECK_SUPPORTED((int64_t)B * nseg <= 65535);
  float* seg_state = nullptr;
  float* seg_dt = nullptr;
  if (seg > 0) {
    if (!workspace || workspace_bytes < cvllm_ssm_scan_workspace_bytes(B, max_new, heads, P, N)) {
      set_last_error("state-space scan workspace too small");
      return CVLLM_E_WORKSPACE;
    }
    seg_state = workspace;
    seg_dt = workspace + (size_t)B * nseg * heads * P * N;
  }
  const dim3 grid(heads, B * nseg, cdiv(P, 2 * PT));
  const int threads = PT * NS;
  // two stages of (B rows, C rows, x rows) + the output rows + step sizes and decays
  const int npt = scan_npt(N);
  const size_t smem = sizeof(float) * ((size_t)2 * kScanTokens * (2 * NS * (npt + kPad) + 2 * PT) +
                                       (size_t)kScanTokens * 2 * PT + 2 * kScanTokens);
  static std::atomic<uint64_t> mask_b[4], mask_f[4];   // per kernel instance: [8 | 16 state channels per thread][with | without output]
#define CVLLM_SCAN(T, MASK, MODE)                                                                                  \
  do {                                                                                                             \
    auto kern = npt == 8 ? (MODE == 1 ? ssm_scan_kernel<T, 8, false> : ssm_scan_kernel<T, 8, true>)                \
                         : (MODE == 1 ? ssm_scan_kernel<T, 16, false> : ssm_scan_kernel<T, 16, true>);                                                                             \
    if (smem > 48 * 1024) CVLLM_CHECK_CUDA(ensure_max_dyn_smem(reinterpret_cast<const void*>(kern), (int)smem, MASK[(npt == 16) * 2 + (MODE == 1)])); \
    kern<<<grid, threads, smem, st>>>(xbc, xbc_stride, static_cast<const T*>(proj), proj_stride, dt_off, dt_bias, A_log, D, \
                                  state, g, y, y_stride, heads, groups, P, N, NS, PT, reserved_slot, MODE, nseg,  \
                                  seg > 0 ? seg : max_new, seg_state, seg_dt);                                     \
    CVLLM_CHECK_LAUNCH();                                                                                          \
  } while (0)
  if (seg <= 0) {
    if (dtype == CVLLM_BF16) CVLLM_SCAN(__nv_bfloat16, mask_b, 0);
    else CVLLM_SCAN(float, mask_f, 0);
    return CVLLM_OK;
  }
  if (dtype == CVLLM_BF16) CVLLM_SCAN(__nv_bfloat16, mask_b, 1);
  else CVLLM_SCAN(float, mask_f, 1);
  ssm_seg_combine_kernel<<<dim3(heads, B), 256, 0, st>>>(seg_state, seg_dt, state, A_log, g, heads, P, N, nseg, seg,
                                                         reserved_slot);
  CVLLM_CHECK_LAUNCH();
  if (dtype == CVLLM_BF16) CVLLM_SCAN(__nv_bfloat16, mask_b, 2);
  else CVLLM_SCAN(float, mask_f, 2);
#undef CVLLM_SCAN
  return CVLLM_OK;
}

extern "C" int cvllm_gated_group_norm(const float* y, int64_t y_stride, const void* z, int64_t z_stride,
                                      const float* weight, float eps, void* out, int64_t out_stride, int64_t rows,
                                      int width, int parts, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(rows >= 0 && width > 0 && parts > 0 && width % parts == 0);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(y && z && weight && out && ssm_dtype_ok(dtype));
  const int part = width / parts;
  const size_t smem = (size_t)part * sizeof(float);
  CVLLM_CHECK_SUPPORTED(smem <= 48 * 1024 && parts <= 65535 && rows <= 2147483647);
  auto st = static_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)rows, parts);
  if (dtype == CVLLM_BF16)
    gated_group_norm_kernel<__nv_bfloat16><<<grid, 128, smem, st>>>(y, y_stride, static_cast<const __nv_bfloat16*>(z),
                                                                    z_stride, weight, eps,
                                                                    static_cast<__nv_bfloat16*>(out), out_stride, part);
  else
    gated_group_norm_kernel<float><<<grid, 128, smem, st>>>(y, y_stride, static_cast<const float*>(z), z_stride, weight,
                                                            eps, static_cast<float*>(out), out_stride, part);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_selective_scan(const void* x, int64_t x_stride, const void* dt_raw, int64_t dt_stride,
                                    const float* dt_bias, const void* bc, int64_t bc_stride, int b_off, int c_off,
                                    const float* A_log, const float* D, const void* z, int64_t z_stride, int z_off,
                                    float* state, const int32_t* cu_seqlens_q, const int32_t* seq_start,
                                    const int32_t* positions, const int32_t* batch_mapping, int B, int max_new,
                                    void* out, int64_t out_stride, int inner, int N, int reserved_slot, int dtype,
                                    cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(B >= 0 && max_new >= 0 && inner > 0 && N > 0);
  if (B == 0 || max_new == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(x && dt_raw && dt_bias && bc && A_log && D && z && state && batch_mapping && out &&
                  ssm_dtype_ok(dtype));
  CVLLM_CHECK_ARG(cu_seqlens_q ? seq_start != nullptr : (positions != nullptr && max_new == 1));
  // state channels per thread: 8 while that fills the SMs with threads, halved down to 1 otherwise (a portion of a few
  // thousand channels has nothing but its channels x N recurrences to run side by side); N <= 32 * NPT
  int npt = 8;
  while (npt > 1 && N <= 32 * (npt / 2) && (int64_t)B * inner * cdiv(N, npt) < (int64_t)sm_count() * 1536) npt >>= 1;
  while (npt < 8 && N > 32 * npt) npt <<= 1;
  int NS = 1;
  while (NS * npt < N) NS <<= 1;
  CVLLM_CHECK_SUPPORTED(NS <= 32 && B <= 65535);
  // up to 256 threads, at most 64 channels a CTA (their staged step sizes, inputs and outputs bound the shared memory)
  int threads = 64 * NS < 256 ? 64 * NS : 256;
  if (threads < 32) threads = 32;
  const int CT = threads / NS;
  auto st = static_cast<cudaStream_t>(stream);
  const StepGeom g{cu_seqlens_q, seq_start, positions, batch_mapping};
  const dim3 grid(cdiv(inner, CT), B);
  const size_t smem = sizeof(float) * (size_t)kSelTokens * (2 * NS * npt + 3 * CT);
  static std::atomic<uint64_t> sel_mask[8];   // per kernel instance: [type][log2 NPT]
#define CVLLM_SEL(T, NPT)                                                                                            \
  do {                                                                                                               \
    if (smem > 48 * 1024)                                                                                            \
      CVLLM_CHECK_CUDA(ensure_max_dyn_smem(reinterpret_cast<const void*>(selective_scan_kernel<T, NPT>), 128 * 1024, \
                                           sel_mask[(sizeof(T) == 2 ? 4 : 0) + (NPT == 1 ? 0 : NPT == 2 ? 1 : NPT == 4 ? 2 : 3)])); \
    selective_scan_kernel<T, NPT><<<grid, threads, smem, st>>>(                                                      \
        static_cast<const T*>(x), x_stride, static_cast<const T*>(dt_raw), dt_stride, dt_bias,                       \
        static_cast<const T*>(bc), bc_stride, b_off, c_off, A_log, D, static_cast<const T*>(z), z_stride, z_off,     \
        state, g, static_cast<T*>(out), out_stride, inner, N, NS, CT, reserved_slot);                                \
  } while (0)
#define CVLLM_SEL_BY_NPT(T)                                                                                          \
  do {                                                                                                               \
    if (npt == 1) CVLLM_SEL(T, 1);                                                                                   \
    else if (npt == 2) CVLLM_SEL(T, 2);                                                                              \
    else if (npt == 4) CVLLM_SEL(T, 4);                                                                              \
    else CVLLM_SEL(T, 8);                                                                                            \
  } while (0)
  if (dtype == CVLLM_BF16) CVLLM_SEL_BY_NPT(__nv_bfloat16);
  else CVLLM_SEL_BY_NPT(float);
#undef CVLLM_SEL_BY_NPT
#undef CVLLM_SEL
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}
