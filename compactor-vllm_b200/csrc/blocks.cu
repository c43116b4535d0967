// Model blocks around the attention path that keep a 32-bit residual stream: sandwich RMS norm
// (post-norm of a branch added into the residual, fused with the pre-norm of the next branch), gated
// activations over packed [gate | up] rows, and a softmax router with group-limited top-k choice.
// Every kernel takes 32-bit or 16-bit activations; norm statistics, softmax and the residual are always 32-bit.
#include "common.cuh"

namespace cvllm {
namespace {

template <typename T>
__device__ __forceinline__ float to_f(T v);
template <>
__device__ __forceinline__ float to_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

constexpr int kThreads = 256;

// sum over the CTA; every thread gets the result.  `red` holds one float per warp.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();  // red may still be read from an earlier call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.f;
  return warp_sum(t);
}

// One CTA per row.  row (dynamic shared memory) holds the row in fp32 between the passes.
//   y != NULL:      resid (+)= y / sqrt(mean(y^2) + eps) * (w_post + gain_offset)      ('=' when assign is set)
//   w_pre != NULL:  out = resid / sqrt(mean(resid^2) + eps) * (w_pre + gain_offset)
//   out != NULL and w_pre == NULL:  out = resid, rounded to the output type
template <typename TY, typename TO>
__global__ void __launch_bounds__(kThreads) sandwich_norm_kernel(
    const TY* __restrict__ y, int64_t y_stride, const float* __restrict__ w_post, float* __restrict__ resid,
    int64_t r_stride, const float* __restrict__ w_pre, TO* __restrict__ out, int64_t o_stride, int width,
    float eps, float gain_offset, int assign) {
  extern __shared__ float row[];
  __shared__ float red[kThreads / 32];
  const int64_t r = blockIdx.x;
  float* res = resid + r * r_stride;
  if (y != nullptr) {
    const TY* yr = y + r * y_stride;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += kThreads) {
      const float v = to_f<TY>(yr[i]);
      row[i] = v;
      ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += kThreads) {
      const float nv = row[i] * inv * (w_post[i] + gain_offset);
      const float v = assign ? nv : res[i] + nv;
      res[i] = v;
      row[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += kThreads) row[i] = res[i];
  }
  if (out == nullptr) return;
  TO* o = out + r * o_stride;
  if (w_pre == nullptr) {   // every thread reads back what it wrote itself
    for (int i = threadIdx.x; i < width; i += kThreads) o[i] = from_f<TO>(row[i]);
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += kThreads) ss += row[i] * row[i];
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += kThreads) o[i] = from_f<TO>(row[i] * inv * (w_pre[i] + gain_offset));
}

// One CTA per row of a 32-bit residual stream:
//   resid += a + b + c     (a, b [rows, width] of type TY, c fp32; each may be NULL)
//   out = norm(resid)      (out may be NULL: the sum alone)
// KIND 0: resid / sqrt(mean(resid^2) + eps) * w;   KIND 1, layer norm: (resid - mean) / sqrt(var + eps) * w + bias with
// var = the mean of the squared deviations (second pass over the row held in shared memory).  Sum, statistics and the
// stream are fp32 whatever the activations' type.
template <typename TY, typename TO, int KIND>
__global__ void __launch_bounds__(kThreads) residual_norm_kernel(
    const TY* __restrict__ a, int64_t a_stride, const TY* __restrict__ b, int64_t b_stride, const float* __restrict__ c,
    int64_t c_stride, float* __restrict__ resid, int64_t r_stride, const float* __restrict__ w,
    const float* __restrict__ bias, TO* __restrict__ out, int64_t o_stride, int width, float eps) {
  extern __shared__ float row[];
  __shared__ float red[kThreads / 32];
  const int64_t r = blockIdx.x;
  float* res = resid + r * r_stride;
  const bool sums = a != nullptr || b != nullptr || c != nullptr;
  float s1 = 0.f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    float v = res[i];
    if (a != nullptr) v += to_f<TY>(a[r * a_stride + i]);
    if (b != nullptr) v += to_f<TY>(b[r * b_stride + i]);
    if (c != nullptr) v += c[r * c_stride + i];
    if (sums) res[i] = v;
    row[i] = v;
    s1 += KIND == 1 ? v : v * v;
  }
  if (out == nullptr) return;
  TO* o = out + r * o_stride;
  s1 = block_sum(s1, red);
  if constexpr (KIND == 0) {
    const float inv = 1.0f / sqrtf(s1 / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += kThreads) o[i] = from_f<TO>(row[i] * inv * w[i]);
  } else {
    const float mean = s1 / (float)width;
    float s2 = 0.f;
    for (int i = threadIdx.x; i < width; i += kThreads) {   // every thread reads back what it wrote itself
      const float d = row[i] - mean;
      s2 += d * d;
    }
    s2 = block_sum(s2, red);
    const float inv = 1.0f / sqrtf(s2 / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += kThreads)
      o[i] = from_f<TO>((row[i] - mean) * inv * w[i] + (bias ? bias[i] : 0.f));
  }
}

// Token embedding plus a hashed embedding of the (previous token, token) pair, one CTA per token:
//   out[t, :] = embed[id_t, :] + pair[row_t, :],   row_t = (prev_t * mul_prev + id_t * mul_cur) mod buckets,
// and row_t = buckets (the table's extra last row) for a sequence's first token (position 0).  prev_t is the token
// before t in the step when that one belongs to the same sequence (same slot, position one less), else the slot's
// entry of prev_state (the last token of the sequence's previous step).  fp32 sum of the two rows.
template <typename T>
__global__ void __launch_bounds__(kThreads) pair_embed_kernel(
    const int64_t* __restrict__ ids, const int32_t* __restrict__ positions, const int32_t* __restrict__ token_slot,
    const T* __restrict__ embed, const T* __restrict__ pair, int64_t buckets, int64_t mul_prev, int64_t mul_cur,
    const int32_t* __restrict__ prev_state, float* __restrict__ out, int64_t o_stride, int width) {
  const int t = blockIdx.x;
  const int64_t id = ids[t];
  const int pos = positions[t], slot = token_slot[t];
  int64_t prow = buckets;
  if (pos > 0) {
    int64_t prev;
    if (t > 0 && token_slot[t - 1] == slot && positions[t - 1] == pos - 1) prev = ids[t - 1];
    else prev = prev_state[slot];
    prow = (prev * mul_prev + id * mul_cur) % buckets;
  }
  const T* e = embed + id * width;
  const T* pr = pair + prow * width;
  float* o = out + (int64_t)t * o_stride;
  for (int i = threadIdx.x; i < width; i += kThreads) o[i] = to_f<T>(e[i]) + to_f<T>(pr[i]);
}

// prev_state[slot] = the last token each sequence brings in this step (runs after pair_embed_kernel has read the old one)
__global__ void pair_state_update_kernel(const int64_t* __restrict__ ids, const int32_t* __restrict__ token_slot,
                                         int32_t* __restrict__ prev_state, int T, int reserved_slot) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const int slot = token_slot[t];
  if (slot == reserved_slot) return;
  if (t == T - 1 || token_slot[t + 1] != slot) prev_state[slot] = (int32_t)ids[t];
}

__device__ __forceinline__ float act_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float act_gelu_tanh(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// KIND 2, the clamped gated unit: g = min(gate, limit), u = clamp(up, -limit, limit), g * sigmoid(1.702 g) * (u + 1)
__device__ __forceinline__ float act_clamped_glu(float g, float u, float limit) {
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.0f + expf(-1.702f * g)) * (u + 1.0f);
}
template <int KIND>
__device__ __forceinline__ float gated(float g, float u, float limit) {
  if constexpr (KIND == 0) return act_silu(g) * u;
  else if constexpr (KIND == 1) return act_gelu_tanh(g) * u;
  else return act_clamped_glu(g, u, limit);
}

// out[t, f] = act(x[t, f]) * x[t, F + f]   (KIND 0 silu, 1 tanh gelu; 2 the clamped gated unit)
template <typename T, int KIND>
__global__ void gated_act_kernel(const T* __restrict__ x, int64_t x_stride, T* __restrict__ out,
                                 int64_t o_stride, int64_t rows, int F, float limit) {
  const int64_t total = rows * (int64_t)F;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / F;
    const int f = (int)(i - t * F);
    const float g = to_f<T>(x[t * x_stride + f]);
    const float u = to_f<T>(x[t * x_stride + F + f]);
    out[t * o_stride + f] = from_f<T>(gated<KIND>(g, u, limit));
  }
}

// the same, eight elements per thread with 16-byte loads (F and both strides multiples of 8, 16-byte aligned bases)
template <typename T, int KIND>
__global__ void gated_act_vec_kernel(const T* __restrict__ x, int64_t x_stride, T* __restrict__ out,
                                     int64_t o_stride, int64_t rows, int F, float limit) {
  const int F8 = F / 8;
  const int64_t total = rows * (int64_t)F8;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / F8;
    const int f = (int)(i - t * F8) * 8;
    float g[8], u[8];
    const T* gp = x + t * x_stride + f;
    T* op = out + t * o_stride + f;
    if constexpr (sizeof(T) == 2) {
      const uint4 a = ldg_nc_v4(gp), b = ldg_nc_v4(gp + F);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        g[2 * k] = __uint_as_float(aw[k] << 16);
        g[2 * k + 1] = __uint_as_float(aw[k] & 0xffff0000u);
        u[2 * k] = __uint_as_float(bw[k] << 16);
        u[2 * k + 1] = __uint_as_float(bw[k] & 0xffff0000u);
      }
      uint32_t r[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float lo = gated<KIND>(g[2 * k], u[2 * k], limit);
        const float hi = gated<KIND>(g[2 * k + 1], u[2 * k + 1], limit);
        r[k] = pack2<true>(lo, hi);
      }
      *reinterpret_cast<uint4*>(op) = make_uint4(r[0], r[1], r[2], r[3]);
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        g[k] = to_f<T>(gp[k]);
        u[k] = to_f<T>(gp[F + k]);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) op[k] = from_f<T>(gated<KIND>(g[k], u[k], limit));
    }
  }
}

// Lowest index among the largest values of v[0..n) (lanes strided), then the same answer in every lane.
__device__ __forceinline__ int warp_argmax(const float* v, int n, float* best_out) {
  const int lane = threadIdx.x & 31;
  float best = -INFINITY;
  int at = 0x7fffffff;
  for (int e = lane; e < n; e += 32) {
    const float c = v[e];
    if (c > best || (c == best && e < at)) { best = c; at = e; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oa = __shfl_xor_sync(0xffffffffu, at, o);
    if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
  }
  *best_out = best;
  return at;
}

constexpr int kRouteWarps = 4;

// One warp per token.  mode 0: s = softmax(logits); choice = s + correction; experts outside the `keep` groups with
// the largest group maximum of choice are struck; the `top` largest remaining choices are taken, each with
// its plain s as weight.  mode 1: the `top` largest LOGITS are taken (lowest index first among equals) and the
// weights are the softmax over the chosen logits alone.  mode 2: the same choice (the largest sigmoid(logit) are the
// largest logits), each with its own sigmoid(logit) as weight, not renormalized.  Shared memory per warp: s[E], choice[E], group maxima[groups].
__global__ void __launch_bounds__(kRouteWarps * 32) route_kernel(
    const float* __restrict__ logits, int64_t l_stride, const float* __restrict__ correction, int T, int E,
    int top, int groups, int keep, int mode, int32_t* __restrict__ idx, float* __restrict__ wts) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * kRouteWarps + warp;
  if (t >= T) return;
  float* s = sm + (size_t)warp * (2 * E + groups);
  float* c = s + E;
  float* gm = c + E;
  const float* z = logits + (int64_t)t * l_stride;
  if (mode == 1 || mode == 2) {
    for (int e = lane; e < E; e += 32) c[e] = z[e];
    __syncwarp();
    float zmax = 0.f, sum = 0.f;
    for (int r = 0; r < top; ++r) {
      float b;
      const int e = warp_argmax(c, E, &b);
      __syncwarp();
      if (r == 0) zmax = b;               // the first choice is the largest logit
      const float p = mode == 2 ? 1.0f / (1.0f + expf(-b)) : expf(b - zmax);
      sum += p;
      if (lane == 0) {
        idx[(int64_t)t * top + r] = e;
        wts[(int64_t)t * top + r] = p;
        c[e] = NAN;
      }
      __syncwarp();
    }
    if (mode == 1 && lane < top) wts[(int64_t)t * top + lane] /= sum;   // top <= 32 in this mode (checked by the host)
    return;
  }
  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(z[e] - m);
    s[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  for (int e = lane; e < E; e += 32) {
    const float p = s[e] / sum;
    s[e] = p;
    c[e] = correction ? p + correction[e] : p;
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int size = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float b = -INFINITY;
      for (int e = g * size; e < (g + 1) * size; ++e) b = fmaxf(b, c[e]);
      gm[g] = b;
    }
    __syncwarp();
    // a kept group's maximum is overwritten with NaN as its mark; experts of unmarked groups are struck afterwards
    for (int r = 0; r < keep; ++r) {
      float b;
      const int g = warp_argmax(gm, groups, &b);
      __syncwarp();
      if (lane == 0) gm[g] = NAN;  // NaN never wins a '>' or '==' comparison again
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (!isnan(gm[e / size])) c[e] = -INFINITY;
    __syncwarp();
  }
  for (int r = 0; r < top; ++r) {
    float b;
    const int e = warp_argmax(c, E, &b);
    __syncwarp();
    if (lane == 0) {
      idx[(int64_t)t * top + r] = e;
      wts[(int64_t)t * top + r] = s[e];
      c[e] = NAN;
    }
    __syncwarp();
  }
}

// out[t, :] = sum_r w[t, r] * (idx[t, r] < n_real ? y[pos[t * top + r], :] : h[t, :])  (+ s_t shared[t, :]),  fp32 sums;
// w == NULL: every weight is 1 (experts whose weight went into their input).
// pos maps a (token, choice) pair to its row of y (the pairs sorted by expert); NULL = the pair's own index.
// s_t = sigmoid(shared_gate[t * gate_stride]) when shared_gate is given (one logit per token), else 1.
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int32_t* __restrict__ pos,
                                   const float* __restrict__ w, int top,
                                   const int32_t* __restrict__ idx, int n_real, const T* __restrict__ h,
                                   const T* __restrict__ shared, const float* __restrict__ shared_gate,
                                   int64_t gate_stride, float* __restrict__ out, int64_t rows, int width) {
  const int64_t total = rows * (int64_t)width;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / width;
    const int c = (int)(i - t * width);
    float acc = shared ? to_f<T>(shared[i]) : 0.f;
    if (shared && shared_gate) acc *= 1.0f / (1.0f + expf(-shared_gate[t * gate_stride]));
    for (int r = 0; r < top; ++r) {
      const float wr = w ? w[t * top + r] : 1.0f;
      if (idx[t * top + r] >= n_real)
        acc += wr * to_f<T>(h[i]);
      else
        acc += wr * to_f<T>(y[(int64_t)(pos ? pos[t * top + r] : t * top + r) * width + c]);
    }
    out[i] = acc;
  }
}


// Expert products for a few tokens (decode): one warp per (pair, output), pair = (token, choice).
//   GATED:  out[p, f] = act(W[e, f, :] . x) * W[e, F + f, :] . x        (W [E, 2F, K])
//   else:   out[p, n] = W[e, n, :] . x                                   (W [E, N, K])
// with e = idx[p] and x = row p / x_div of xs.  Pairs whose expert is >= n_real (identity experts) are skipped.
// No host knowledge of the routing is needed, so the step can be replayed from a CUDA graph.
template <typename T, bool GATED, int KIND>
__global__ void __launch_bounds__(256) expert_gemv_kernel(const T* __restrict__ xs, int x_div,
                                                          const T* __restrict__ w, const int32_t* __restrict__ idx,
                                                          int n_real, T* __restrict__ out, int N, int K,
                                                          float limit) {
  const int p = blockIdx.y;
  const int e = idx[p];
  if (e >= n_real) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * 8 + warp;
  if (n >= N) return;
  const T* x = xs + (int64_t)(p / x_div) * K;
  const int rows = GATED ? 2 * N : N;
  const T* w0 = w + ((int64_t)e * rows + n) * K;
  float a = 0.f, b = 0.f;
  for (int k = lane; k < K; k += 32) {
    const float xv = to_f<T>(x[k]);
    a = fmaf(to_f<T>(w0[k]), xv, a);
    if (GATED) b = fmaf(to_f<T>(w0[(int64_t)N * K + k]), xv, b);
  }
  a = warp_sum(a);
  if (GATED) {
    b = warp_sum(b);
    // the library GEMM path rounds gate and up to the storage type before the activation; do the same
    a = to_f<T>(from_f<T>(a));
    b = to_f<T>(from_f<T>(b));
    a = gated<KIND>(a, b, limit);
  }
  if (lane == 0) out[(int64_t)p * N + n] = from_f<T>(a);
}

// One CTA per row of a 32-bit residual stream, for layers whose sublayer outputs pass a gate on the way in:
//   resid += sigmoid(gate) * y      (y of type TY, gate logits of type TG, both [rows, width]; y == NULL: no sum)
//   out = resid / sqrt(mean(resid^2) + eps) * w          (out == NULL: the sum alone)
// i.e. the gated residual sum of one sublayer fused with the RMS norm in front of the next.
template <typename TY, typename TG, typename TO>
__global__ void __launch_bounds__(kThreads) gated_residual_norm_kernel(
    const TY* __restrict__ y, int64_t y_stride, const TG* __restrict__ gate, int64_t g_stride,
    float* __restrict__ resid, int64_t r_stride, const float* __restrict__ w, TO* __restrict__ out, int64_t o_stride,
    int width, float eps) {
  extern __shared__ float row[];
  __shared__ float red[kThreads / 32];
  const int64_t r = blockIdx.x;
  float* res = resid + r * r_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    float v = res[i];
    if (y != nullptr) {
      const float gz = to_f<TG>(gate[r * g_stride + i]);
      v = fmaf(1.0f / (1.0f + expf(-gz)), to_f<TY>(y[r * y_stride + i]), v);
      res[i] = v;
    }
    row[i] = v;
    ss += v * v;
  }
  if (out == nullptr) return;
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)width + eps);
  TO* o = out + r * o_stride;
  for (int i = threadIdx.x; i < width; i += kThreads) o[i] = from_f<TO>(row[i] * inv * w[i]);
}

// One CTA per row: out = scale * (a / rms(a) * wa + b / rms(b) * wb), rms(v) = sqrt(mean(v^2) + eps) - two branch
// outputs, each RMS-normed with a weight of its own, blended.  Statistics and the sum are fp32.
template <typename T>
__global__ void __launch_bounds__(kThreads) dual_norm_blend_kernel(const T* __restrict__ a, int64_t a_stride,
                                                                   const float* __restrict__ wa,
                                                                   const T* __restrict__ b, int64_t b_stride,
                                                                   const float* __restrict__ wb, T* __restrict__ out,
                                                                   int64_t o_stride, int width, float eps, float scale) {
  __shared__ float red[kThreads / 32];
  const int64_t r = blockIdx.x;
  float sa = 0.f, sb = 0.f;
  for (int i = threadIdx.x; i < width; i += kThreads) {
    const float va = to_f<T>(a[r * a_stride + i]), vb = to_f<T>(b[r * b_stride + i]);
    sa += va * va;
    sb += vb * vb;
  }
  sa = block_sum(sa, red);
  sb = block_sum(sb, red);
  const float ia = scale / sqrtf(sa / (float)width + eps), ib = scale / sqrtf(sb / (float)width + eps);
  for (int i = threadIdx.x; i < width; i += kThreads)
    out[r * o_stride + i] = from_f<T>(to_f<T>(a[r * a_stride + i]) * ia * wa[i] + to_f<T>(b[r * b_stride + i]) * ib * wb[i]);
}

// Plain activations of one tensor.  KIND 0: relu(x)^2.
template <typename T, int KIND>
__global__ void unary_act_kernel(const T* __restrict__ x, int64_t x_stride, T* __restrict__ out, int64_t o_stride,
                                 int64_t rows, int F) {
  const int64_t total = rows * (int64_t)F;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / F;
    const int f = (int)(i - t * F);
    const float v = fmaxf(to_f<T>(x[t * x_stride + f]), 0.f);
    out[t * o_stride + f] = from_f<T>(v * v);
  }
}

// out[t, c] = cap * tanh(x[t, c] / cap), fp32 out
template <typename T>
__global__ void softcap_kernel(const T* __restrict__ x, int64_t x_stride, float* __restrict__ out, int64_t o_stride,
                               int64_t rows, int F, float cap) {
  const int64_t total = rows * (int64_t)F;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / F;
    const int f = (int)(i - t * F);
    out[t * o_stride + f] = cap * tanhf(to_f<T>(x[t * x_stride + f]) / cap);
  }
}

// out[p, :] = x[pair / top, :] * scale[pair], pair = perm ? perm[p] : p - the rows of (token, choice) pairs, each
// multiplied by its routing weight on the way into its expert (rounded to the activations' type).
template <typename T>
__global__ void scaled_rows_kernel(const T* __restrict__ x, int64_t x_stride, const int64_t* __restrict__ perm,
                                   const float* __restrict__ scale, int top, T* __restrict__ out, int64_t pairs,
                                   int width) {
  const int64_t total = pairs * (int64_t)width;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t p = i / width;
    const int c = (int)(i - p * width);
    const int64_t pair = perm ? perm[p] : p;
    out[i] = from_f<T>(to_f<T>(x[(pair / top) * x_stride + c]) * scale[pair]);
  }
}

}  // namespace
}  // namespace cvllm

using namespace cvllm;

extern "C" int cvllm_sandwich_norm(const void* y, int64_t y_stride, int y_dtype, const float* w_post, float* resid,
                                   int64_t r_stride, const float* w_pre, void* out, int64_t o_stride,
                                   int out_dtype, int rows, int width, float eps, float gain_offset, int assign,
                                   cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(rows >= 0 && width > 0 && resid);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG((y == nullptr) == (w_post == nullptr));
  CVLLM_CHECK_ARG(w_pre == nullptr || out != nullptr);
  CVLLM_CHECK_ARG(!assign || y != nullptr);
  CVLLM_CHECK_ARG(y == nullptr || y_dtype == CVLLM_BF16 || y_dtype == CVLLM_F32);
  CVLLM_CHECK_ARG(out == nullptr || out_dtype == CVLLM_BF16 || out_dtype == CVLLM_F32);
  CVLLM_CHECK_SUPPORTED(width <= 12288);
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)width * sizeof(float);
  const bool yb = y_dtype == CVLLM_BF16, ob = out_dtype == CVLLM_BF16;
#define CVLLM_SANDWICH(TY, TO)                                                                                 \
  sandwich_norm_kernel<TY, TO><<<rows, kThreads, smem, st>>>(static_cast<const TY*>(y), y_stride, w_post,      \
                                                             resid, r_stride, w_pre, static_cast<TO*>(out),    \
                                                             o_stride, width, eps, gain_offset, assign)
  if (yb && ob) CVLLM_SANDWICH(__nv_bfloat16, __nv_bfloat16);
  else if (yb) CVLLM_SANDWICH(__nv_bfloat16, float);
  else if (ob) CVLLM_SANDWICH(float, __nv_bfloat16);
  else CVLLM_SANDWICH(float, float);
#undef CVLLM_SANDWICH
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_residual_norm(const void* a, int64_t a_stride, const void* b, int64_t b_stride, int ab_dtype,
                                   const float* c, int64_t c_stride, float* resid, int64_t r_stride, const float* w,
                                   const float* bias, void* out, int64_t o_stride, int out_dtype, int rows, int width,
                                   float eps, int kind, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(rows >= 0 && width > 0 && resid && (kind == 0 || kind == 1));
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG((a == nullptr && b == nullptr) || ab_dtype == CVLLM_BF16 || ab_dtype == CVLLM_F32);
  CVLLM_CHECK_ARG(out == nullptr || (w != nullptr && (out_dtype == CVLLM_BF16 || out_dtype == CVLLM_F32)));
  CVLLM_CHECK_SUPPORTED(width <= 12288);
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)width * sizeof(float);
  const bool yb = ab_dtype == CVLLM_BF16 && (a || b), ob = out_dtype == CVLLM_BF16;
#define CVLLM_RESNORM(TY, TO, KIND)                                                                                \
  residual_norm_kernel<TY, TO, KIND><<<rows, kThreads, smem, st>>>(                                                \
      static_cast<const TY*>(a), a_stride, static_cast<const TY*>(b), b_stride, c, c_stride, resid, r_stride, w,    \
      bias, static_cast<TO*>(out), o_stride, width, eps)
#define CVLLM_RESNORM_K(TY, TO) \
  do { if (kind == 0) CVLLM_RESNORM(TY, TO, 0); else CVLLM_RESNORM(TY, TO, 1); } while (0)
  if (yb && ob) CVLLM_RESNORM_K(__nv_bfloat16, __nv_bfloat16);
  else if (yb) CVLLM_RESNORM_K(__nv_bfloat16, float);
  else if (ob) CVLLM_RESNORM_K(float, __nv_bfloat16);
  else CVLLM_RESNORM_K(float, float);
#undef CVLLM_RESNORM_K
#undef CVLLM_RESNORM
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_pair_hash_embed(const int64_t* ids, const int32_t* positions, const int32_t* token_slot,
                                     const void* embed, const void* pair, int64_t buckets, int64_t mul_prev,
                                     int64_t mul_cur, int32_t* prev_state, float* out, int64_t out_stride, int T,
                                     int width, int reserved_slot, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(T >= 0 && width > 0 && buckets > 0);
  if (T == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(ids && positions && token_slot && embed && pair && prev_state && out);
  CVLLM_CHECK_ARG(dtype == CVLLM_BF16 || dtype == CVLLM_F32);
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == CVLLM_BF16)
    pair_embed_kernel<__nv_bfloat16><<<T, kThreads, 0, st>>>(ids, positions, token_slot,
                                                             static_cast<const __nv_bfloat16*>(embed),
                                                             static_cast<const __nv_bfloat16*>(pair), buckets, mul_prev,
                                                             mul_cur, prev_state, out, out_stride, width);
  else
    pair_embed_kernel<float><<<T, kThreads, 0, st>>>(ids, positions, token_slot, static_cast<const float*>(embed),
                                                     static_cast<const float*>(pair), buckets, mul_prev, mul_cur,
                                                     prev_state, out, out_stride, width);
  pair_state_update_kernel<<<cdiv(T, 256), 256, 0, st>>>(ids, token_slot, prev_state, T, reserved_slot);
  CVLLM_CHECK_LAUNCHES(2);
  return CVLLM_OK;
}

extern "C" int cvllm_gated_act(const void* x, int64_t x_stride, void* out, int64_t o_stride, int64_t rows, int F,
                               int kind, float limit, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(rows >= 0 && F > 0 && kind >= 0 && kind <= 2);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(x && out && (dtype == CVLLM_BF16 || dtype == CVLLM_F32));
  auto st = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * (int64_t)F;
  const int grid = (int)((total + 255) / 256 < (int64_t)sm_count() * 16 ? (total + 255) / 256 : (int64_t)sm_count() * 16);
  const bool vec = F % 8 == 0 && x_stride % 8 == 0 && o_stride % 8 == 0 && aligned16(x) && aligned16(out);
#define CVLLM_GATED(T, K)                                                                                      \
  if (vec)                                                                                                     \
    gated_act_vec_kernel<T, K><<<(grid + 7) / 8, 256, 0, st>>>(static_cast<const T*>(x), x_stride,             \
                                                               static_cast<T*>(out), o_stride, rows, F, limit); \
  else                                                                                                         \
    gated_act_kernel<T, K><<<grid, 256, 0, st>>>(static_cast<const T*>(x), x_stride, static_cast<T*>(out),     \
                                                 o_stride, rows, F, limit)
  if (dtype == CVLLM_BF16) {
    if (kind == 0) { CVLLM_GATED(__nv_bfloat16, 0); } else if (kind == 1) { CVLLM_GATED(__nv_bfloat16, 1); }
    else { CVLLM_GATED(__nv_bfloat16, 2); }
  } else {
    if (kind == 0) { CVLLM_GATED(float, 0); } else if (kind == 1) { CVLLM_GATED(float, 1); }
    else { CVLLM_GATED(float, 2); }
  }
#undef CVLLM_GATED
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_moe_route(const float* logits, int64_t l_stride, const float* correction, int T, int E, int top,
                               int groups, int keep, int mode, int32_t* idx, float* wts, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(T >= 0 && E > 0 && top > 0 && top <= E && groups > 0 && keep > 0 && keep <= groups);
  CVLLM_CHECK_ARG(mode == 0 || ((mode == 1 || mode == 2) && groups == 1 && correction == nullptr));
  CVLLM_CHECK_SUPPORTED(mode == 0 || top <= 32);
  if (T == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(logits && idx && wts && E % groups == 0 && keep * (E / groups) >= top);
  CVLLM_CHECK_SUPPORTED(E <= 2048);
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)kRouteWarps * (2 * E + groups) * sizeof(float);
  static std::atomic<uint64_t> mask{0};
  if (smem > 48 * 1024)
    CVLLM_CHECK_CUDA(ensure_max_dyn_smem(reinterpret_cast<const void*>(route_kernel), (int)smem, mask));
  route_kernel<<<cdiv(T, kRouteWarps), kRouteWarps * 32, smem, st>>>(logits, l_stride, correction, T, E, top,
                                                                    groups, keep, mode, idx, wts);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_moe_combine(const void* y, const int32_t* pos, const float* w, int top, const int32_t* idx, int n_real,
                                 const void* h, const void* shared, const float* shared_gate, int64_t gate_stride,
                                 float* out, int64_t rows, int width, int dtype, cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(rows >= 0 && width > 0 && top > 0);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(y && idx && h && out && (dtype == CVLLM_BF16 || dtype == CVLLM_F32));
  auto st = static_cast<cudaStream_t>(stream);
  const int64_t total = rows * (int64_t)width;
  const int grid = (int)((total + 255) / 256 < (int64_t)sm_count() * 16 ? (total + 255) / 256 : (int64_t)sm_count() * 16);
  if (dtype == CVLLM_BF16)
    moe_combine_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        static_cast<const __nv_bfloat16*>(y), pos, w, top, idx, n_real, static_cast<const __nv_bfloat16*>(h),
        static_cast<const __nv_bfloat16*>(shared), shared_gate, gate_stride, out, rows, width);
  else
    moe_combine_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(y), pos, w, top, idx, n_real,
                                                    static_cast<const float*>(h), static_cast<const float*>(shared),
                                                    shared_gate, gate_stride, out, rows, width);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_expert_gemv(const void* xs, int x_div, const void* w, const int32_t* idx, int n_real, void* out,
                                 int pairs, int N, int K, int gated_kind, float limit, int dtype,
                                 cvllm_stream_t stream) {
  CVLLM_CHECK_ARG(pairs >= 0 && N > 0 && K > 0 && x_div > 0 && gated_kind >= -1 && gated_kind <= 2);
  if (pairs == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(xs && w && idx && out && (dtype == CVLLM_BF16 || dtype == CVLLM_F32));
  CVLLM_CHECK_SUPPORTED(pairs <= 65535);
  auto st = static_cast<cudaStream_t>(stream);
  dim3 grid(cdiv(N, 8), pairs);
#define CVLLM_GEMV(T, G, KD)                                                                                   \
  expert_gemv_kernel<T, G, KD><<<grid, 256, 0, st>>>(static_cast<const T*>(xs), x_div, static_cast<const T*>(w), \
                                                     idx, n_real, static_cast<T*>(out), N, K, limit)
  if (dtype == CVLLM_BF16) {
    if (gated_kind < 0) CVLLM_GEMV(__nv_bfloat16, false, 0);
    else if (gated_kind == 0) CVLLM_GEMV(__nv_bfloat16, true, 0);
    else if (gated_kind == 1) CVLLM_GEMV(__nv_bfloat16, true, 1);
    else CVLLM_GEMV(__nv_bfloat16, true, 2);
  } else {
    if (gated_kind < 0) CVLLM_GEMV(float, false, 0);
    else if (gated_kind == 0) CVLLM_GEMV(float, true, 0);
    else if (gated_kind == 1) CVLLM_GEMV(float, true, 1);
    else CVLLM_GEMV(float, true, 2);
  }
#undef CVLLM_GEMV
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

static int block_grid(int64_t total) {
  const int64_t want = (total + 255) / 256, cap = (int64_t)sm_count() * 16;
  return (int)(want < cap ? want : cap);
}

extern "C" int cvllm_gated_residual_norm(const void* y, int64_t y_stride, int y_dtype, const void* gate,
                                         int64_t g_stride, int g_dtype, float* resid, int64_t r_stride, const float* w,
                                         void* out, int64_t o_stride, int out_dtype, int rows, int width, float eps,
                                         cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(rows >= 0 && width > 0 && resid);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG((y == nullptr) == (gate == nullptr));
  CVLLM_CHECK_ARG(y == nullptr || ((y_dtype == CVLLM_BF16 || y_dtype == CVLLM_F32) &&
                                   (g_dtype == CVLLM_BF16 || g_dtype == CVLLM_F32)));
  CVLLM_CHECK_ARG(out == nullptr || (w != nullptr && (out_dtype == CVLLM_BF16 || out_dtype == CVLLM_F32)));
  CVLLM_CHECK_SUPPORTED(width <= 12288);
  auto st = static_cast<cudaStream_t>(stream);
  const size_t smem = (size_t)width * sizeof(float);
  const bool yb = y && y_dtype == CVLLM_BF16, gb = y && g_dtype == CVLLM_BF16, ob = out && out_dtype == CVLLM_BF16;
#define CVLLM_GRN(TY, TG, TO)                                                                                       \
  gated_residual_norm_kernel<TY, TG, TO><<<rows, kThreads, smem, st>>>(                                             \
      static_cast<const TY*>(y), y_stride, static_cast<const TG*>(gate), g_stride, resid, r_stride, w,              \
      static_cast<TO*>(out), o_stride, width, eps)
  if (yb && gb && ob) CVLLM_GRN(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
  else if (yb && gb) CVLLM_GRN(__nv_bfloat16, __nv_bfloat16, float);
  else if (gb && ob) CVLLM_GRN(float, __nv_bfloat16, __nv_bfloat16);
  else if (gb) CVLLM_GRN(float, __nv_bfloat16, float);
  else if (ob) CVLLM_GRN(float, float, __nv_bfloat16);
  else if (!yb) CVLLM_GRN(float, float, float);
  else { set_last_error("gated_residual_norm: 16-bit branch with 32-bit gate"); return CVLLM_E_UNSUPPORTED; }
#undef CVLLM_GRN
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_dual_norm_blend(const void* a, int64_t a_stride, const float* wa, const void* b, int64_t b_stride,
                                     const float* wb, void* out, int64_t o_stride, int rows, int width, float eps,
                                     float scale, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(rows >= 0 && width > 0);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(a && wa && b && wb && out && (dtype == CVLLM_BF16 || dtype == CVLLM_F32));
  auto st = static_cast<cudaStream_t>(stream);
  if (dtype == CVLLM_BF16)
    dual_norm_blend_kernel<__nv_bfloat16><<<rows, kThreads, 0, st>>>(
        static_cast<const __nv_bfloat16*>(a), a_stride, wa, static_cast<const __nv_bfloat16*>(b), b_stride, wb,
        static_cast<__nv_bfloat16*>(out), o_stride, width, eps, scale);
  else
    dual_norm_blend_kernel<float><<<rows, kThreads, 0, st>>>(static_cast<const float*>(a), a_stride, wa,
                                                             static_cast<const float*>(b), b_stride, wb,
                                                             static_cast<float*>(out), o_stride, width, eps, scale);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_unary_act(const void* x, int64_t x_stride, void* out, int64_t o_stride, int64_t rows, int F,
                               int kind, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(rows >= 0 && F > 0 && kind == 0);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(x && out && (dtype == CVLLM_BF16 || dtype == CVLLM_F32));
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = block_grid(rows * (int64_t)F);
  if (dtype == CVLLM_BF16)
    unary_act_kernel<__nv_bfloat16, 0><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), x_stride,
                                                             static_cast<__nv_bfloat16*>(out), o_stride, rows, F);
  else
    unary_act_kernel<float, 0><<<grid, 256, 0, st>>>(static_cast<const float*>(x), x_stride, static_cast<float*>(out),
                                                     o_stride, rows, F);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_softcap(const void* x, int64_t x_stride, float* out, int64_t o_stride, int64_t rows, int F,
                             float cap, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(rows >= 0 && F > 0 && cap > 0.f);
  if (rows == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(x && out && (dtype == CVLLM_BF16 || dtype == CVLLM_F32));
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = block_grid(rows * (int64_t)F);
  if (dtype == CVLLM_BF16)
    softcap_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), x_stride, out, o_stride,
                                                        rows, F, cap);
  else
    softcap_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), x_stride, out, o_stride, rows, F, cap);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}

extern "C" int cvllm_scaled_rows(const void* x, int64_t x_stride, const int64_t* perm, const float* scale, int top,
                                 void* out, int64_t pairs, int width, int dtype, cvllm_stream_t stream) {
  drop_stale_error();
  CVLLM_CHECK_ARG(pairs >= 0 && width > 0 && top > 0);
  if (pairs == 0) return CVLLM_OK;
  CVLLM_CHECK_ARG(x && scale && out && (dtype == CVLLM_BF16 || dtype == CVLLM_F32));
  auto st = static_cast<cudaStream_t>(stream);
  const int grid = block_grid(pairs * (int64_t)width);
  if (dtype == CVLLM_BF16)
    scaled_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(x), x_stride, perm, scale,
                                                            top, static_cast<__nv_bfloat16*>(out), pairs, width);
  else
    scaled_rows_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(x), x_stride, perm, scale, top,
                                                    static_cast<float*>(out), pairs, width);
  CVLLM_CHECK_LAUNCH();
  return CVLLM_OK;
}
