// seq_ops.cu -- the row-wise kernels around the sequence mixers of the hybrid decoders:
//
//   residual_rmsnorm     h = norm(r)                      r: the fp32 residual stream
//   residual_add_norms   r += norm_post(y); h = norm_pre(r)      one pass, both reductions in the CTA
//   causal_conv          short depth-wise convolution over time with a per-sequence tail carried in a slot
//   unitnorm_temp_cache  per-head unit RMS of q and k, position-dependent query temperature, K/V scatter
//   gated_norm           (grouped) RMS norm and an output gate, in either order
//   act_and_mul          act(gate) * up for the gated feed-forward
//   act_only             act(x) for a feed-forward without a gate (silu, relu, gelu, squared relu)
//   norm_residual        r (+)= norm(y [+ y2]); h = r in the element type: a norm on the sublayer's OUTPUT (layer norm
//                        with weight and bias, or RMS norm), the rows of y / y2 optionally gathered by index
//                        (token embedding + learned position + norm in one launch)
//   rownorm_cache        RMS norm of q and of k over the WHOLE projection (all heads at once), K/V scatter
//   gate_prep            what a gated linear recurrence with tied input reads: silu(q) and the lower-bounded forget
//                        gate l + (1 - l) sigmoid(f + bias), both fp32
//   gather_rows_by_head  cache (or packed) rows picked by slot, written per kv head: [entries, G, keys, size] -- the
//                        operand layout of attention composed of batched products
//   residual_scale_groupnorm  r (+)= c * scale[channel] * y (rows of y optionally gathered by index: the scaled token
//                        embedding); h = RMS norm of r in equal consecutive groups, times a weight
//   rotary_table         cos / sin of position * frequency for a table of frequencies (fp64 angles), times a magnitude
//   rope_mix_cache       rotation of part of every q and k head by that table, values blended with another layer's
//                        values of the same token, K/V scatter
//   head_gate            every head of a row times sigmoid of one logit per (token, head)
//
// All are bound by HBM traffic; arithmetic is fp32 whatever the element type. Shapes are free: no
// multiple-of-8 rule, so that small and odd models run (a 16-byte path is taken where rows allow it).
#include "seq_common.cuh"

namespace b200 {

// ------------------------------------------------------------------ norms over the fp32 residual
// weight w is stored as the deviation from `offset`: y = x * rsqrt(mean x^2 + eps) * (offset + w)
template <typename T>
__global__ void __launch_bounds__(256)
residual_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ res, const float* __restrict__ w,
                        float offset, float eps, int hidden) {
  __shared__ float red[32];
  pdl_wait();
  const float* r = res + (int64_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) ss += r[i] * r[i];
  const float rstd = 1.0f / sqrtf(cta_sum(ss, red) / (float)hidden + eps);
  T* o = out + (int64_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(r[i] * rstd * (offset + w[i]));
}

// r <- r + norm(y; w_post);  h <- norm(r; w_pre)  (h skipped when w_pre == nullptr). Dynamic smem: hidden floats.
template <typename T>
__global__ void __launch_bounds__(256)
residual_add_norms_kernel(T* __restrict__ h, float* __restrict__ res, const T* __restrict__ y,
                          const float* __restrict__ w_post, const float* __restrict__ w_pre, float offset,
                          float eps, int hidden) {
  extern __shared__ float row[];
  __shared__ float red[32];
  pdl_wait();
  const T* yr = y + (int64_t)blockIdx.x * hidden;
  float* r = res + (int64_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = to_f32<T>(yr[i]);
    row[i] = v;
    ss += v * v;
  }
  const float rstd = 1.0f / sqrtf(cta_sum(ss, red) / (float)hidden + eps);
  float ss2 = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = r[i] + row[i] * rstd * (offset + w_post[i]);
    r[i] = v;
    row[i] = v;
    ss2 += v * v;
  }
  if (w_pre == nullptr) return;
  const float rstd2 = 1.0f / sqrtf(cta_sum(ss2, red) / (float)hidden + eps);
  T* o = h + (int64_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_f32<T>(row[i] * rstd2 * (offset + w_pre[i]));
}

// 16-byte form of the two kernels above (hidden % 8 == 0): a thread keeps its 8-element vectors of the row in
// registers (up to kResVecs per thread, 256 threads: hidden <= 8192), so the row is read once. The CTA has one
// thread per vector up to 256, so that narrow rows do not idle half of it.
constexpr int kResVecs = 4;

template <typename T>
__global__ void __launch_bounds__(256)
residual_add_norms_vec_kernel(T* __restrict__ h, float* __restrict__ res, const T* __restrict__ y,
                              const float* __restrict__ w_post, const float* __restrict__ w_pre, float offset,
                              float eps, int hidden) {
  __shared__ float red[32];
  pdl_wait();
  const int nvec = hidden / 8;
  const T* yr = y + (int64_t)blockIdx.x * hidden;
  float* r = res + (int64_t)blockIdx.x * hidden;
  float val[kResVecs][8];
  float ss = 0.f;
#pragma unroll
  for (int n = 0; n < kResVecs; ++n) {
    const int vi = threadIdx.x + n * blockDim.x;
    if (vi < nvec) {
      load8<T>(yr + vi * 8, val[n]);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += val[n][e] * val[n][e];
    }
  }
  const float rstd = 1.0f / sqrtf(cta_sum(ss, red) / (float)hidden + eps);
  float ss2 = 0.f;
#pragma unroll
  for (int n = 0; n < kResVecs; ++n) {
    const int vi = threadIdx.x + n * blockDim.x;
    if (vi < nvec) {
      float rv[8], wv[8];
      load8<float>(r + vi * 8, rv);
      load8<float>(w_post + vi * 8, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        val[n][e] = rv[e] + val[n][e] * rstd * (offset + wv[e]);
        ss2 += val[n][e] * val[n][e];
      }
      store8<float>(r + vi * 8, val[n]);
    }
  }
  if (w_pre == nullptr) return;
  const float rstd2 = 1.0f / sqrtf(cta_sum(ss2, red) / (float)hidden + eps);
  T* o = h + (int64_t)blockIdx.x * hidden;
#pragma unroll
  for (int n = 0; n < kResVecs; ++n) {
    const int vi = threadIdx.x + n * blockDim.x;
    if (vi < nvec) {
      float wv[8], ov[8];
      load8<float>(w_pre + vi * 8, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) ov[e] = val[n][e] * rstd2 * (offset + wv[e]);
      store8<T>(o + vi * 8, ov);
    }
  }
}

// ------------------------------------------------------------------ causal convolution over time
// out[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c]), u = 0 before the sequence's start.
// The last taps-1 inputs of every sequence live in state[slot] as [taps-1, C] (oldest first) between steps.
// One thread = one channel x kConvSeg consecutive tokens of one sequence. Only the thread of a sequence's
// first segment reads the carried tail, and the same thread writes the new one (from the chunk's last rows,
// which it reads itself), so no other thread can see a half-updated tail.
constexpr int kConvSeg = 16;
constexpr int kConvMaxTaps = 16;

template <typename T>
__global__ void __launch_bounds__(128)
causal_conv_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ x, int64_t x_stride,
                   const float* __restrict__ w, const float* __restrict__ bias, int act, T* __restrict__ state,
                   const int* __restrict__ state_slots, const int* __restrict__ cu_q,
                   const int* __restrict__ cu_k, const int* __restrict__ ctx_lens, int C, int taps) {
  pdl_wait();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int s = blockIdx.z;
  const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
  const int t0 = blockIdx.y * kConvSeg;
  if (c >= C || t0 >= sp.q_len) return;
  const int hist = taps - 1;
  const bool carried = state != nullptr && sp.first_pos() > 0;
  T* tail = state != nullptr ? state + (int64_t)state_slots[s] * hist * C : nullptr;

  float wt[kConvMaxTaps];
#pragma unroll
  for (int j = 0; j < kConvMaxTaps; ++j) wt[j] = j < taps ? w[(int64_t)c * taps + j] : 0.f;
  const float b = bias != nullptr ? bias[c] : 0.f;

  // input at token index i of this chunk (negative: the carried tail, or zeros at a sequence's start)
  auto input = [&](int i) -> float {
    if (i >= 0) return to_f32<T>(x[(int64_t)(sp.q_start + i) * x_stride + c]);
    return carried ? to_f32<T>(tail[(int64_t)(hist + i) * C + c]) : 0.f;
  };
  float win[kConvMaxTaps];   // win[j] multiplies wt[j]; win[taps-1] is the current token
#pragma unroll
  for (int j = 0; j < kConvMaxTaps; ++j) win[j] = (j >= 1 && j < taps) ? input(t0 - taps + j) : 0.f;
  // (win[1 .. taps-1] now hold inputs t0-taps+1 .. t0-1; the loop shifts before it loads)
  const int t1 = min(t0 + kConvSeg, sp.q_len);
  for (int t = t0; t < t1; ++t) {
#pragma unroll
    for (int j = 0; j < kConvMaxTaps - 1; ++j) win[j] = win[j + 1];
    const float cur = input(t);
#pragma unroll
    for (int j = 0; j < kConvMaxTaps; ++j)
      if (j == taps - 1) win[j] = cur;
    float acc = b;
#pragma unroll
    for (int j = 0; j < kConvMaxTaps; ++j)
      if (j < taps) acc += wt[j] * win[j];
    if (act == 1) acc = silu_f(acc);
    out[(int64_t)(sp.q_start + t) * out_stride + c] = from_f32<T>(acc);
  }
  if (t0 == 0 && tail != nullptr && hist > 0) {
    float keep[kConvMaxTaps];
#pragma unroll
    for (int j = 0; j < kConvMaxTaps; ++j) keep[j] = j < hist ? input(sp.q_len - hist + j) : 0.f;
#pragma unroll
    for (int j = 0; j < kConvMaxTaps; ++j)
      if (j < hist) tail[(int64_t)j * C + c] = from_f32<T>(keep[j]);
  }
}

// 16-byte form (channels, strides % 8 == 0): one thread = 8 channels x kConvSeg tokens, same ownership of the tail
template <typename T, int MT>
__global__ void __launch_bounds__(128)
causal_conv_vec_kernel(T* __restrict__ out, int64_t out_stride, const T* __restrict__ x, int64_t x_stride,
                       const float* __restrict__ w, const float* __restrict__ bias, int act, T* __restrict__ state,
                       const int* __restrict__ state_slots, const int* __restrict__ cu_q,
                       const int* __restrict__ cu_k, const int* __restrict__ ctx_lens, int C, int taps) {
  pdl_wait();
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  const int s = blockIdx.z;
  const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
  const int t0 = blockIdx.y * kConvSeg;
  if (c >= C || t0 >= sp.q_len) return;
  const int hist = taps - 1;
  const bool carried = state != nullptr && sp.first_pos() > 0;
  T* tail = state != nullptr ? state + (int64_t)state_slots[s] * hist * C : nullptr;
  float wt[MT][8], b[8];
#pragma unroll
  for (int j = 0; j < MT; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) wt[j][e] = j < taps ? w[(int64_t)(c + e) * taps + j] : 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) b[e] = bias != nullptr ? bias[c + e] : 0.f;
  auto input = [&](int i, float (&f)[8]) {
    if (i >= 0) {
      load8<T>(x + (int64_t)(sp.q_start + i) * x_stride + c, f);
    } else if (carried) {
      load8<T>(tail + (int64_t)(hist + i) * C + c, f);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
  };
  float win[MT][8];
#pragma unroll
  for (int j = 0; j < MT; ++j) {
    if (j >= 1 && j < taps) {
      input(t0 - taps + j, win[j]);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) win[j][e] = 0.f;
    }
  }
  const int t1 = min(t0 + kConvSeg, sp.q_len);
  for (int t = t0; t < t1; ++t) {
    float cur[8], acc[8];
    input(t, cur);
#pragma unroll
    for (int j = 0; j < MT - 1; ++j)
#pragma unroll
      for (int e = 0; e < 8; ++e) win[j][e] = win[j + 1][e];
#pragma unroll
    for (int j = 0; j < MT; ++j)
      if (j == taps - 1) {
#pragma unroll
        for (int e = 0; e < 8; ++e) win[j][e] = cur[e];
      }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = b[e];
#pragma unroll
    for (int j = 0; j < MT; ++j)
      if (j < taps) {
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[e] += wt[j][e] * win[j][e];
      }
    if (act == 1) {
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] = silu_f(acc[e]);
    }
    store8<T>(out + (int64_t)(sp.q_start + t) * out_stride + c, acc);
  }
  if (t0 == 0 && tail != nullptr && hist > 0) {
    float keep[MT][8];
#pragma unroll
    for (int j = 0; j < MT; ++j)
      if (j < hist) input(sp.q_len - hist + j, keep[j]);
#pragma unroll
    for (int j = 0; j < MT; ++j)
      if (j < hist) store8<T>(tail + (int64_t)j * C + c, keep[j]);
  }
}

// ------------------------------------------------------------------ q/k unit norm, query temperature, K/V scatter
// qkv: [T, H*dim | G*dim | G*vdim] (row stride given). Per head: q <- q / rms(q) * temp(pos), k <- k / rms(k),
// temp(p) = 1 + coef * ln(floor((p + 1) / every) + 1). q and k are rewritten in place; k and v are also
// stored at their cache slot when caches are bound. One warp per (token, head of q | k | v).
template <typename T>
__global__ void __launch_bounds__(256)
unitnorm_temp_cache_kernel(T* __restrict__ qkv, int64_t stride, const int64_t* __restrict__ positions,
                           float eps, float coef, int every, T* __restrict__ k_cache, T* __restrict__ v_cache,
                           const int* __restrict__ slots, int slot_pairs, int block_size, int num_tokens,
                           int H, int G, int dim, int vdim) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int per_tok = H + 2 * G;
  if (unit >= (int64_t)num_tokens * per_tok) return;
  const int t = (int)(unit / per_tok), u = (int)(unit % per_tok);
  int64_t slot = -1;
  if (k_cache != nullptr && u >= H) {
    slot = slot_pairs ? (int64_t)slots[2 * t] * block_size + slots[2 * t + 1] : (int64_t)slots[t];
    if (slot < 0) return;
  }
  T* row = qkv + (int64_t)t * stride;
  if (u >= H + G) {                                  // a value head: copy only
    const int g = u - H - G;
    if (k_cache == nullptr) return;
    const T* src = row + (int64_t)H * dim + (int64_t)G * dim + (int64_t)g * vdim;
    T* dst = v_cache + slot * ((int64_t)G * vdim) + (int64_t)g * vdim;
    for (int i = lane; i < vdim; i += 32) dst[i] = src[i];
    return;
  }
  T* x = row + (int64_t)u * dim;                     // q heads then k heads, both `dim` wide
  float ss = 0.f;
  for (int i = lane; i < dim; i += 32) {
    const float v = to_f32<T>(x[i]);
    ss += v * v;
  }
  float mul = 1.0f / sqrtf(warp_sum(ss) / (float)dim + eps);
  if (u < H) {
    const int64_t steps = (positions[t] + 1) / every;
    mul *= 1.0f + coef * logf((float)steps + 1.0f);
  }
  T* dst = (u >= H && k_cache != nullptr) ? k_cache + slot * ((int64_t)G * dim) + (int64_t)(u - H) * dim : nullptr;
  for (int i = lane; i < dim; i += 32) {
    const T v = from_f32<T>(to_f32<T>(x[i]) * mul);
    x[i] = v;
    if (dst != nullptr) dst[i] = v;
  }
}

// 16-byte form: dim = 8 * GL with GL a power of two; GL adjacent lanes share one head, 32 / GL heads per warp
template <typename T, int GL>
__global__ void __launch_bounds__(256)
unitnorm_temp_cache_vec_kernel(T* __restrict__ qkv, int64_t stride, const int64_t* __restrict__ positions,
                               float eps, float coef, int every, T* __restrict__ k_cache, T* __restrict__ v_cache,
                               const int* __restrict__ slots, int slot_pairs, int block_size, int num_tokens,
                               int H, int G, int vdim) {
  pdl_wait();
  constexpr int dim = GL * 8, UPW = 32 / GL;
  const int lane = threadIdx.x & 31, gl = lane % GL;
  const int64_t unit = ((int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * UPW + lane / GL;
  const int per_tok = H + 2 * G;
  const bool live = unit < (int64_t)num_tokens * per_tok;
  const int t = live ? (int)(unit / per_tok) : 0, u = live ? (int)(unit % per_tok) : 0;
  int64_t slot = -1;
  if (live && k_cache != nullptr && u >= H)
    slot = slot_pairs ? (int64_t)slots[2 * t] * block_size + slots[2 * t + 1] : (int64_t)slots[t];
  T* row = qkv + (int64_t)t * stride;
  const bool is_v = u >= H + G;
  if (live && is_v && slot >= 0) {
    const T* src = row + (int64_t)(H + G) * dim + (int64_t)(u - H - G) * vdim;
    T* dst = v_cache + slot * ((int64_t)G * vdim) + (int64_t)(u - H - G) * vdim;
    for (int vi = gl; vi * 8 < vdim; vi += GL) {
      float tmp[8];
      load8<T>(src + vi * 8, tmp);
      store8<T>(dst + vi * 8, tmp);
    }
  }
  const bool normed = live && !is_v;
  T* x = row + (int64_t)u * dim + gl * 8;
  float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (normed) load8<T>(x, f);
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
#pragma unroll
  for (int off = GL / 2; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  if (!normed) return;
  float mul = 1.0f / sqrtf(ss / (float)dim + eps);
  if (u < H) {
    const int64_t steps = (positions[t] + 1) / every;
    mul *= 1.0f + coef * logf((float)steps + 1.0f);
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) f[e] *= mul;
  store8<T>(x, f);
  if (u >= H && slot >= 0) store8<T>(k_cache + slot * ((int64_t)G * dim) + (int64_t)(u - H) * dim + gl * 8, f);
}

// ------------------------------------------------------------------ gated (grouped) RMS norm
// y: [rows, n] fp32 or T; gate: [rows, n] T with a row stride. One CTA per (row, group of n / groups):
//   gate_first: out = norm_group(y * act(gate)) * w          (gate, then norm)
//   else      : out = norm_group(y) * w * act(gate)          (norm, then gate)
// w == nullptr: no norm at all, out = y * act(gate). gate_act: 0 sigmoid, 1 silu, 2 no gate (gate may be null).
template <typename T, typename Y>
__global__ void __launch_bounds__(256)
gated_norm_kernel(T* __restrict__ out, const Y* __restrict__ y, const T* __restrict__ gate,
                  int64_t gate_stride, const float* __restrict__ w, float eps, int n, int groups,
                  int gate_first, int gate_act) {
  __shared__ float red[32];
  pdl_wait();
  const int64_t r = blockIdx.x;
  const int len = n / groups, lo = blockIdx.y * len;
  const Y* yr = y + r * n + lo;
  const T* gr = gate + r * gate_stride + lo;
  T* o = out + r * n + lo;
  auto gate_at = [&](int i) -> float {
    if (gate_act == 2) return 1.f;
    const float g = to_f32<T>(gr[i]);
    return gate_act == 1 ? silu_f(g) : sigmoid_f(g);
  };
  if (w == nullptr) {
    for (int i = threadIdx.x; i < len; i += blockDim.x) o[i] = from_f32<T>(to_f32<Y>(yr[i]) * gate_at(i));
    return;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < len; i += blockDim.x) {
    float v = to_f32<Y>(yr[i]);
    if (gate_first) v *= gate_at(i);
    ss += v * v;
  }
  const float rstd = 1.0f / sqrtf(cta_sum(ss, red) / (float)len + eps);
  for (int i = threadIdx.x; i < len; i += blockDim.x) {
    float v = to_f32<Y>(yr[i]);
    if (gate_first) v = v * gate_at(i) * rstd * w[lo + i];
    else v = v * rstd * w[lo + i] * gate_at(i);
    o[i] = from_f32<T>(v);
  }
}

// ------------------------------------------------------------------ act(gate) * up
// x: [rows, 2 * inter] (gate | up) -> out [rows, inter]. act: 0 silu, 1 relu, 2 gelu (tanh form).
template <typename T>
__global__ void __launch_bounds__(256)
act_and_mul_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int inter, int act) {
  pdl_wait();
  const int64_t total = rows * inter;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / inter;
    const int c = (int)(i - r * inter);
    const float g = to_f32<T>(x[r * 2 * inter + c]), u = to_f32<T>(x[r * 2 * inter + inter + c]);
    const float a = act == 1 ? fmaxf(g, 0.f) : act == 2 ? gelu_tanh_f(g) : silu_f(g);
    out[i] = from_f32<T>(a * u);
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
act_and_mul_vec_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int inter8, int act) {
  pdl_wait();
  const int64_t total = rows * inter8;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / inter8;
    const int c = (int)(i - r * inter8);
    float g[8], u[8], o[8];
    load8<T>(x + (r * 2 * inter8 + c) * 8, g);
    load8<T>(x + (r * 2 * inter8 + inter8 + c) * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float a = act == 1 ? fmaxf(g[e], 0.f) : act == 2 ? gelu_tanh_f(g[e]) : silu_f(g[e]);
      o[e] = a * u[e];
    }
    store8<T>(out + i * 8, o);
  }
}

// 16-byte form of gated_norm (n / groups % 8 == 0): one CTA per (row, group), 8 elements per thread and step
template <typename T, typename Y>
__global__ void __launch_bounds__(256)
gated_norm_vec_kernel(T* __restrict__ out, const Y* __restrict__ y, const T* __restrict__ gate,
                      int64_t gate_stride, const float* __restrict__ w, float eps, int n, int groups,
                      int gate_first, int gate_act) {
  __shared__ float red[32];
  pdl_wait();
  const int64_t r = blockIdx.x;
  const int len = n / groups, lo = blockIdx.y * len;
  const Y* yr = y + r * n + lo;
  const T* gr = gate + r * gate_stride + lo;
  T* o = out + r * n + lo;
  constexpr int kV = 2;                               // up to 256 * 2 * 8 = 4096 elements per group in registers
  float val[kV][8], gv[kV][8];
  float ss = 0.f;
#pragma unroll
  for (int m = 0; m < kV; ++m) {
    const int vi = threadIdx.x + m * blockDim.x;
    if (vi * 8 < len) {
      load8<Y>(yr + vi * 8, val[m]);
      if (gate_act != 2) load8<T>(gr + vi * 8, gv[m]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        gv[m][e] = gate_act == 2 ? 1.f : gate_act == 1 ? silu_f(gv[m][e]) : sigmoid_f(gv[m][e]);
        if (gate_first || w == nullptr) val[m][e] *= gv[m][e];
        ss += val[m][e] * val[m][e];
      }
    }
  }
  float rstd = 1.f;
  if (w != nullptr) rstd = 1.0f / sqrtf(cta_sum(ss, red) / (float)len + eps);
#pragma unroll
  for (int m = 0; m < kV; ++m) {
    const int vi = threadIdx.x + m * blockDim.x;
    if (vi * 8 < len) {
      float ov[8];
      if (w != nullptr) {
        float wv[8];
        load8<float>(w + lo + vi * 8, wv);
#pragma unroll
        for (int e = 0; e < 8; ++e) ov[e] = gate_first ? val[m][e] * rstd * wv[e] : val[m][e] * rstd * wv[e] * gv[m][e];
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) ov[e] = val[m][e];
      }
      store8<T>(o + vi * 8, ov);
    }
  }
}

// groups of at most 512 elements (one norm per head): GL = 1 .. 32 adjacent lanes per (row, group) -- the smallest power
// of two that covers the group with 8 elements per lane (two steps per lane above 256 elements) -- so that every lane of
// a warp works; sums by xor shuffles inside the lane group, no shared memory
template <typename T, typename Y>
__global__ void __launch_bounds__(256)
gated_norm_warp_kernel(T* __restrict__ out, const Y* __restrict__ y, const T* __restrict__ gate,
                       int64_t gate_stride, const float* __restrict__ w, float eps, int64_t rows, int n, int groups,
                       int gate_first, int gate_act, int gl) {
  pdl_wait();
  const int lane = threadIdx.x & 31, sub = lane % gl;
  const int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int64_t unit = warp * (32 / gl) + lane / gl;
  const bool live = unit < rows * groups;
  const int64_t r = live ? unit / groups : 0;
  const int len = n / groups, lo = live ? (int)(unit % groups) * len : 0;
  const Y* yr = y + r * n + lo;
  const T* gr = gate + r * gate_stride + lo;
  T* o = out + r * n + lo;
  constexpr int kV = 2;
  float val[kV][8], gv[kV][8];
  float ss = 0.f;
#pragma unroll
  for (int m = 0; m < kV; ++m) {
    const int vi = sub + m * gl;
    if (live && vi * 8 < len && (m == 0 || gl == 32)) {
      load8<Y>(yr + vi * 8, val[m]);
      if (gate_act != 2) load8<T>(gr + vi * 8, gv[m]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        gv[m][e] = gate_act == 2 ? 1.f : gate_act == 1 ? silu_f(gv[m][e]) : sigmoid_f(gv[m][e]);
        if (gate_first) val[m][e] *= gv[m][e];
        ss += val[m][e] * val[m][e];
      }
    }
  }
  for (int off = gl >> 1; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
  const float rstd = 1.0f / sqrtf(ss / (float)len + eps);
#pragma unroll
  for (int m = 0; m < kV; ++m) {
    const int vi = sub + m * gl;
    if (live && vi * 8 < len && (m == 0 || gl == 32)) {
      float ov[8], wv[8];
      load8<float>(w + lo + vi * 8, wv);
#pragma unroll
      for (int e = 0; e < 8; ++e) ov[e] = gate_first ? val[m][e] * rstd * wv[e] : val[m][e] * rstd * wv[e] * gv[m][e];
      store8<T>(o + vi * 8, ov);
    }
  }
}

// ------------------------------------------------------------------ act(x) without a gate
// act: 0 silu, 1 relu, 2 gelu (tanh form), 3 squared relu.
__device__ __forceinline__ float act_f(float x, int act) {
  if (act == 1) return fmaxf(x, 0.f);
  if (act == 2) return gelu_tanh_f(x);
  if (act == 3) {
    const float r = fmaxf(x, 0.f);
    return r * r;
  }
  return silu_f(x);
}

template <typename T>
__global__ void __launch_bounds__(256)
act_only_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t total, int act) {
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x)
    out[i] = from_f32<T>(act_f(to_f32<T>(x[i]), act));
}

template <typename T>
__global__ void __launch_bounds__(256)
act_only_vec_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t total8, int act) {
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total8; i += (int64_t)gridDim.x * blockDim.x) {
    float v[8];
    load8<T>(x + i * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = act_f(v[e], act);
    store8<T>(out + i * 8, v);
  }
}

// ------------------------------------------------------------------ a norm on the sublayer's output, then the residual
// u = y[iy] (+ y2[iy2]) in fp32; n = norm(u): kind 0 (u - mean) / sqrt(var + eps) * w + b, kind 1 u / sqrt(mean u^2 + eps)
// * (offset + w); r <- accumulate ? r + n : n; h <- r in the element type (h may be null). iy / iy2: row r itself, or
// index[r] clamped to the table's rows (a token id, a position). Dynamic smem: hidden floats.
template <typename T>
__global__ void __launch_bounds__(256)
norm_residual_kernel(T* __restrict__ h, float* __restrict__ res, const T* __restrict__ y,
                     const int64_t* __restrict__ y_index, int64_t y_rows, const T* __restrict__ y2,
                     const int64_t* __restrict__ y2_index, int64_t y2_rows, const float* __restrict__ w,
                     const float* __restrict__ b, float eps, float offset, int kind, int accumulate, int hidden) {
  extern __shared__ float row[];
  __shared__ float red[32];
  pdl_wait();
  const int64_t r = blockIdx.x;
  int64_t iy = y_index != nullptr ? y_index[r] : r;
  if (y_index != nullptr) iy = iy < 0 ? 0 : (iy >= y_rows ? y_rows - 1 : iy);
  const T* yr = y + iy * hidden;
  const T* y2r = nullptr;
  if (y2 != nullptr) {
    int64_t i2 = y2_index != nullptr ? y2_index[r] : r;
    if (y2_index != nullptr) i2 = i2 < 0 ? 0 : (i2 >= y2_rows ? y2_rows - 1 : i2);
    y2r = y2 + i2 * hidden;
  }
  float s1 = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = to_f32<T>(yr[i]);
    if (y2r != nullptr) v += to_f32<T>(y2r[i]);
    row[i] = v;
    s1 += kind == 0 ? v : v * v;
  }
  s1 = cta_sum(s1, red) / (float)hidden;
  float mean = 0.f, rstd;
  if (kind == 0) {
    mean = s1;
    float sq = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = row[i] - mean;
      sq += d * d;
    }
    rstd = 1.0f / sqrtf(cta_sum(sq, red) / (float)hidden + eps);
  } else {
    rstd = 1.0f / sqrtf(s1 + eps);
  }
  float* rr = res + r * hidden;
  T* hr = h != nullptr ? h + r * hidden : nullptr;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float n = kind == 0 ? (row[i] - mean) * rstd * w[i] + (b != nullptr ? b[i] : 0.f) : row[i] * rstd * (offset + w[i]);
    if (accumulate) n += rr[i];
    rr[i] = n;
    if (hr != nullptr) hr[i] = from_f32<T>(n);
  }
}

// 16-byte form (hidden % 8 == 0, hidden <= 8 * 256 * kResVecs): a thread keeps its 8-element vectors in registers,
// the row is read once; mean and variance from one pass over registers each.
template <typename T>
__global__ void __launch_bounds__(256)
norm_residual_vec_kernel(T* __restrict__ h, float* __restrict__ res, const T* __restrict__ y,
                         const int64_t* __restrict__ y_index, int64_t y_rows, const T* __restrict__ y2,
                         const int64_t* __restrict__ y2_index, int64_t y2_rows, const float* __restrict__ w,
                         const float* __restrict__ b, float eps, float offset, int kind, int accumulate, int hidden) {
  __shared__ float red[32];
  pdl_wait();
  const int nvec = hidden / 8;
  const int64_t r = blockIdx.x;
  int64_t iy = y_index != nullptr ? y_index[r] : r;
  if (y_index != nullptr) iy = iy < 0 ? 0 : (iy >= y_rows ? y_rows - 1 : iy);
  const T* yr = y + iy * hidden;
  const T* y2r = nullptr;
  if (y2 != nullptr) {
    int64_t i2 = y2_index != nullptr ? y2_index[r] : r;
    if (y2_index != nullptr) i2 = i2 < 0 ? 0 : (i2 >= y2_rows ? y2_rows - 1 : i2);
    y2r = y2 + i2 * hidden;
  }
  float val[kResVecs][8];
  float s1 = 0.f;
#pragma unroll
  for (int n = 0; n < kResVecs; ++n) {
    const int vi = threadIdx.x + n * blockDim.x;
    if (vi < nvec) {
      load8<T>(yr + vi * 8, val[n]);
      if (y2r != nullptr) {
        float t[8];
        load8<T>(y2r + vi * 8, t);
#pragma unroll
        for (int e = 0; e < 8; ++e) val[n][e] += t[e];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) s1 += kind == 0 ? val[n][e] : val[n][e] * val[n][e];
    }
  }
  s1 = cta_sum(s1, red) / (float)hidden;
  float mean = 0.f, rstd;
  if (kind == 0) {
    mean = s1;
    float sq = 0.f;
#pragma unroll
    for (int n = 0; n < kResVecs; ++n) {
      const int vi = threadIdx.x + n * blockDim.x;
      if (vi < nvec) {
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float d = val[n][e] - mean;
          sq += d * d;
        }
      }
    }
    rstd = 1.0f / sqrtf(cta_sum(sq, red) / (float)hidden + eps);
  } else {
    rstd = 1.0f / sqrtf(s1 + eps);
  }
  float* rr = res + r * hidden;
  T* hr = h != nullptr ? h + r * hidden : nullptr;
#pragma unroll
  for (int n = 0; n < kResVecs; ++n) {
    const int vi = threadIdx.x + n * blockDim.x;
    if (vi < nvec) {
      float wv[8], bv[8], ov[8];
      load8<float>(w + vi * 8, wv);
      if (kind == 0 && b != nullptr) load8<float>(b + vi * 8, bv);
      if (accumulate) load8<float>(rr + vi * 8, ov);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float nrm = kind == 0 ? (val[n][e] - mean) * rstd * wv[e] + (b != nullptr ? bv[e] : 0.f)
                                    : val[n][e] * rstd * (offset + wv[e]);
        ov[e] = accumulate ? ov[e] + nrm : nrm;
      }
      store8<float>(rr + vi * 8, ov);
      if (hr != nullptr) store8<T>(hr + vi * 8, ov);
    }
  }
}

// ------------------------------------------------------------------ q / k RMS norm over the whole projection + K/V scatter
// One CTA per (token, part): part 0 = the nq query columns, 1 = the nk key columns, 2 = the nv value columns of row
// x [nq | nk | nv]. q and k are divided by the root mean square of ALL their columns (every head at once), times a
// plain weight, in place; k and v rows go to the paged caches at the token's slot (slot < 0: not stored).
template <typename T>
__global__ void __launch_bounds__(128)
rownorm_cache_kernel(T* __restrict__ x, int64_t stride, const float* __restrict__ wq, const float* __restrict__ wk,
                     float eps, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ slots,
                     int slot_pairs, int block_size, int nq, int nk, int nv) {
  __shared__ float red[32];
  pdl_wait();
  const int64_t t = blockIdx.x;
  const int part = blockIdx.y;
  int64_t slot = -1;
  if (k_cache != nullptr && part > 0)
    slot = slot_pairs ? (int64_t)slots[2 * t] * block_size + slots[2 * t + 1] : (int64_t)slots[t];
  T* row = x + t * stride;
  if (part == 2) {
    if (slot < 0) return;
    const T* src = row + nq + nk;
    T* dst = v_cache + slot * nv;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) dst[i] = src[i];
    return;
  }
  const int n = part == 0 ? nq : nk;
  T* p = row + (part == 0 ? 0 : nq);
  const float* w = part == 0 ? wq : wk;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_f32<T>(p[i]);
    ss += v * v;
  }
  const float rstd = 1.0f / sqrtf(cta_sum(ss, red) / (float)n + eps);
  T* dst = (part == 1 && slot >= 0) ? k_cache + slot * nk : nullptr;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const T v = from_f32<T>(to_f32<T>(p[i]) * rstd * w[i]);
    p[i] = v;
    if (dst != nullptr) dst[i] = v;
  }
}

// 16-byte form (nq, nk, nv, stride % 8 == 0): ONE WARP per (token, part), 8 per CTA -- a part is a few hundred to a few
// thousand elements, too little for a CTA and its barriers. Two passes over the part (the second is served by L1), sums
// by shuffles.
template <typename T>
__global__ void __launch_bounds__(256)
rownorm_cache_vec_kernel(T* __restrict__ x, int64_t stride, const float* __restrict__ wq, const float* __restrict__ wk,
                         float eps, T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ slots,
                         int slot_pairs, int block_size, int num_tokens, int parts, int nq, int nk, int nv) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (unit >= (int64_t)num_tokens * parts) return;
  const int64_t t = unit / parts;
  const int part = (int)(unit % parts);
  int64_t slot = -1;
  if (k_cache != nullptr && part > 0)
    slot = slot_pairs ? (int64_t)slots[2 * t] * block_size + slots[2 * t + 1] : (int64_t)slots[t];
  T* row = x + t * stride;
  if (part == 2) {
    if (slot < 0) return;
    const uint4* src = reinterpret_cast<const uint4*>(row + nq + nk);
    uint4* dst = reinterpret_cast<uint4*>(v_cache + slot * nv);
    for (int i = lane; i < nv * (int)sizeof(T) / 16; i += 32) dst[i] = src[i];
    return;
  }
  const int n = part == 0 ? nq : nk, nvec = n / 8;
  T* p = row + (part == 0 ? 0 : nq);
  const float* w = part == 0 ? wq : wk;
  float ss = 0.f;
  for (int vi = lane; vi < nvec; vi += 32) {
    float v[8];
    load8<T>(p + vi * 8, v);
#pragma unroll
    for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
  }
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)n + eps);
  T* dst = (part == 1 && slot >= 0) ? k_cache + slot * nk : nullptr;
  for (int vi = lane; vi < nvec; vi += 32) {
    float v[8], wv[8];
    load8<T>(p + vi * 8, v);
    load8<float>(w + vi * 8, wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= rstd * wv[e];
    store8<T>(p + vi * 8, v);
    if (dst != nullptr) store8<T>(dst + vi * 8, v);
  }
}

// ------------------------------------------------------------------ inputs of a gated recurrence with tied input
// q32 = silu(q), f32 = l + (1 - l) sigmoid(f + bias): the gate and everything derived from it stay in 32-bit
template <typename T>
__global__ void __launch_bounds__(256)
gate_prep_kernel(float* __restrict__ q_out, float* __restrict__ f_out, const T* __restrict__ q, int64_t q_stride,
                 const T* __restrict__ f, int64_t f_stride, const float* __restrict__ bias,
                 const float* __restrict__ lower, int64_t tokens, int n) {
  pdl_wait();
  const int64_t total = tokens * n;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = i / n;
    const int c = (int)(i - t * n);
    q_out[i] = silu_f(to_f32<T>(q[t * q_stride + c]));
    const float l = lower != nullptr ? lower[c] : 0.f;
    f_out[i] = l + (1.0f - l) * sigmoid_f(to_f32<T>(f[t * f_stride + c]) + (bias != nullptr ? bias[c] : 0.f));
  }
}

// ------------------------------------------------------------------ rows by slot, regrouped per kv head
// out[n][g][j][:] = src[slots[n * nk + j]][g][:] in 16-byte vectors (vph per head): one pass, no index arithmetic on
// the host, the layout that a batched product per kv head reads.
__global__ void __launch_bounds__(256)
gather_rows_by_head_kernel(uint4* __restrict__ out, const char* __restrict__ src, int64_t src_stride_bytes,
                           const int64_t* __restrict__ slots, int64_t total, int nk, int G, int vph) {
  pdl_wait();
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int v = (int)(i % vph);
    const int64_t r = i / vph;
    const int j = (int)(r % nk);
    const int64_t ng = r / nk;
    const int g = (int)(ng % G);
    const int64_t n = ng / G;
    const int64_t slot = slots[n * nk + j];
    out[i] = *reinterpret_cast<const uint4*>(src + slot * src_stride_bytes + ((int64_t)g * vph + v) * 16);
  }
}

// ------------------------------------------------------------------ scaled residual add + grouped RMS norm
// r <- (accumulate ? r : 0) + c * scale[i] * y[i]   (scale == nullptr: c alone; y == nullptr: r unchanged; y_index: row
// t of y is y[clamp(y_index[t])], a table lookup);  h <- r / sqrt(mean over the element's group of r^2 + eps) *
// (offset + w)   (skipped when w == nullptr). The row is split into `groups` equal consecutive parts.
// Dynamic smem: hidden + groups floats. Group sums are taken by one warp per group in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
residual_scale_groupnorm_kernel(T* __restrict__ h, float* __restrict__ res, const T* __restrict__ y,
                                const int64_t* __restrict__ y_index, int64_t y_rows, const float* __restrict__ scale,
                                float c, int accumulate, const float* __restrict__ w, float offset, float eps,
                                int hidden, int groups) {
  extern __shared__ float row[];                     // [hidden] then rstd [groups]
  float* rstd = row + hidden;
  pdl_wait();
  float* r = res + (int64_t)blockIdx.x * hidden;
  const T* yr = nullptr;
  if (y != nullptr) {
    int64_t src = blockIdx.x;
    if (y_index != nullptr) src = min(max(y_index[blockIdx.x], (int64_t)0), y_rows - 1);
    yr = y + src * hidden;
  }
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = accumulate ? r[i] : 0.f;
    if (yr != nullptr) {
      const float u = c * (scale != nullptr ? scale[i] : 1.0f);
      v += u * to_f32<T>(yr[i]);
      r[i] = v;
    }
    row[i] = v;
  }
  if (w == nullptr) return;
  __syncthreads();
  const int per = hidden / groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g < groups; g += nw) {
    float ss = 0.f;
    for (int i = lane; i < per; i += 32) ss += row[g * per + i] * row[g * per + i];
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = 1.0f / sqrtf(ss / (float)per + eps);
  }
  __syncthreads();
  T* o = h + (int64_t)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) o[i] = from_f32<T>(row[i] * rstd[i / per] * (offset + w[i]));
}

// 16-byte form (hidden % 8 == 0, group size % 8 == 0, hidden <= 8 * 256 * kResVecs): the row stays in registers; every
// 8-element vector leaves its sum of squares in shared memory, one warp per group adds them in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
residual_scale_groupnorm_vec_kernel(T* __restrict__ h, float* __restrict__ res, const T* __restrict__ y,
                                    const int64_t* __restrict__ y_index, int64_t y_rows,
                                    const float* __restrict__ scale, float c, int accumulate,
                                    const float* __restrict__ w, float offset, float eps, int hidden, int groups) {
  __shared__ float part[256 * kResVecs];
  __shared__ float rstd[256];
  pdl_wait();
  const int nvec = hidden / 8;
  float* r = res + (int64_t)blockIdx.x * hidden;
  const T* yr = nullptr;
  if (y != nullptr) {
    int64_t src = blockIdx.x;
    if (y_index != nullptr) src = min(max(y_index[blockIdx.x], (int64_t)0), y_rows - 1);
    yr = y + src * hidden;
  }
  float val[kResVecs][8];
#pragma unroll
  for (int n = 0; n < kResVecs; ++n) {
    const int vi = threadIdx.x + n * blockDim.x;
    if (vi < nvec) {
      if (accumulate) {
        load8<float>(r + vi * 8, val[n]);
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) val[n][e] = 0.f;
      }
      if (yr != nullptr) {
        float yv[8], sv[8];
        load8<T>(yr + vi * 8, yv);
        if (scale != nullptr) {
          load8<float>(scale + vi * 8, sv);
#pragma unroll
          for (int e = 0; e < 8; ++e) val[n][e] += (c * sv[e]) * yv[e];
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) val[n][e] += c * yv[e];
        }
        store8<float>(r + vi * 8, val[n]);
      }
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += val[n][e] * val[n][e];
      part[vi] = ss;
    }
  }
  if (w == nullptr) return;
  __syncthreads();
  const int vper = nvec / groups;                    // vectors per group
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int g = warp; g < groups; g += nw) {
    float ss = 0.f;
    for (int i = lane; i < vper; i += 32) ss += part[g * vper + i];
    ss = warp_sum(ss);
    if (lane == 0) rstd[g] = 1.0f / sqrtf(ss / (float)(vper * 8) + eps);
  }
  __syncthreads();
  T* o = h + (int64_t)blockIdx.x * hidden;
#pragma unroll
  for (int n = 0; n < kResVecs; ++n) {
    const int vi = threadIdx.x + n * blockDim.x;
    if (vi < nvec) {
      float wv[8], ov[8];
      load8<float>(w + vi * 8, wv);
      const float rs = rstd[vi / vper];
#pragma unroll
      for (int e = 0; e < 8; ++e) ov[e] = val[n][e] * rs * (offset + wv[e]);
      store8<T>(o + vi * 8, ov);
    }
  }
}

// ------------------------------------------------------------------ rotary positions from a table of frequencies
// table[t][i] = (cos, sin)(positions[t] * freq[i]) * magnitude: fp64 angle (a position times a frequency loses digits
// in fp32 at long range), fp32 result. Computed once per step for all layers that share the frequencies.
__global__ void __launch_bounds__(256)
rotary_table_kernel(float2* __restrict__ table, const int64_t* __restrict__ positions, const double* __restrict__ freq,
                    double magnitude, int tokens, int half) {
  pdl_wait();
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (int64_t)tokens * half) return;
  const int t = (int)(e / half), i = (int)(e % half);
  double sn, cs;
  sincos((double)positions[t] * freq[i], &sn, &cs);
  table[e] = make_float2((float)(cs * magnitude), (float)(sn * magnitude));
}

// qkv: [T, H*dim | G*dim | G*vdim] (row stride given), rewritten in place. Every q and k head: the first `dims`
// columns are rotated by the table, in pairs (2i, 2i+1) (interleaved) or (i, i + dims/2); the rest pass. Every value
// head: v <- (1 - lambda) v + lambda v_other (lambda a device scalar; skipped when v_other == nullptr). k and v rows are
// also stored at their cache slot when caches are bound. One warp per (token, head of q | k | v); fp32 arithmetic.
template <typename T>
__global__ void __launch_bounds__(256)
rope_mix_cache_kernel(T* __restrict__ qkv, int64_t stride, const float2* __restrict__ table, int dims, int interleaved,
                      const T* __restrict__ v_other, int64_t v_other_stride, const float* __restrict__ lambda,
                      T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ slots, int slot_pairs,
                      int block_size, int num_tokens, int H, int G, int dim, int vdim) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int per_tok = H + 2 * G;
  if (unit >= (int64_t)num_tokens * per_tok) return;
  const int t = (int)(unit / per_tok), u = (int)(unit % per_tok);
  int64_t slot = -1;
  if (k_cache != nullptr && u >= H) {
    slot = slot_pairs ? (int64_t)slots[2 * t] * block_size + slots[2 * t + 1] : (int64_t)slots[t];
    if (slot < 0) k_cache = nullptr, v_cache = nullptr;      // a row without a cache slot is still rewritten in place
  }
  T* row = qkv + (int64_t)t * stride;
  if (u >= H + G) {                                  // a value head
    const int g = u - H - G;
    T* x = row + (int64_t)(H + G) * dim + (int64_t)g * vdim;
    T* dst = v_cache != nullptr ? v_cache + slot * ((int64_t)G * vdim) + (int64_t)g * vdim : nullptr;
    if (v_other == nullptr) {
      if (dst != nullptr)
        for (int i = lane; i < vdim; i += 32) dst[i] = x[i];
      return;
    }
    const float lam = *lambda;
    const T* o = v_other + (int64_t)t * v_other_stride + (int64_t)g * vdim;
    for (int i = lane; i < vdim; i += 32) {
      const T v = from_f32<T>((1.0f - lam) * to_f32<T>(x[i]) + lam * to_f32<T>(o[i]));
      x[i] = v;
      if (dst != nullptr) dst[i] = v;
    }
    return;
  }
  T* x = row + (int64_t)u * dim;                     // q heads then k heads, both `dim` wide
  T* dst = (u >= H && k_cache != nullptr) ? k_cache + slot * ((int64_t)G * dim) + (int64_t)(u - H) * dim : nullptr;
  const int half = dims / 2;
  const float2* cs = table + (int64_t)t * half;
  for (int i = lane; i < half; i += 32) {
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
    const float2 r = cs[i];
    const float p = to_f32<T>(x[a]), q = to_f32<T>(x[b]);
    const T ra = from_f32<T>(p * r.x - q * r.y), rb = from_f32<T>(q * r.x + p * r.y);
    x[a] = ra, x[b] = rb;
    if (dst != nullptr) dst[a] = ra, dst[b] = rb;
  }
  if (dst != nullptr)
    for (int i = dims + lane; i < dim; i += 32) dst[i] = x[i];
}

// 16-byte form of rope_mix_cache (neighbouring pairs; dim, vdim, dims multiples of 8; 16-byte aligned rows): one thread
// per 8 consecutive columns of a token's row, which lie in one head and either inside or outside its rotated part.
template <typename T>
__global__ void __launch_bounds__(256)
rope_mix_cache_vec_kernel(T* __restrict__ qkv, int64_t stride, const float2* __restrict__ table, int dims,
                          const T* __restrict__ v_other, int64_t v_other_stride, const float* __restrict__ lambda,
                          T* __restrict__ k_cache, T* __restrict__ v_cache, const int* __restrict__ slots,
                          int slot_pairs, int block_size, int num_tokens, int H, int G, int dim, int vdim) {
  pdl_wait();
  const int nq = H * dim, nk = G * dim, nv = G * vdim;
  const int vecs = (nq + nk + nv) / 8;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= (int64_t)num_tokens * vecs) return;
  const int t = (int)(e / vecs), c = (int)(e % vecs) * 8;
  T* x = qkv + (int64_t)t * stride + c;
  int64_t slot = -1;
  if (k_cache != nullptr && c >= nq)
    slot = slot_pairs ? (int64_t)slots[2 * t] * block_size + slots[2 * t + 1] : (int64_t)slots[t];
  float f[8];
  if (c >= nq + nk) {                                // a value vector
    const int cv = c - nq - nk;
    if (v_other == nullptr && slot < 0) return;
    load8<T>(x, f);
    if (v_other != nullptr) {
      float o[8];
      load8<T>(v_other + (int64_t)t * v_other_stride + cv, o);
      const float lam = *lambda;
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = (1.0f - lam) * f[i] + lam * o[i];
      store8<T>(x, f);
      load8<T>(x, f);                                // what is cached is exactly what the row now holds
    }
    if (slot >= 0) store8<T>(v_cache + slot * (int64_t)nv + cv, f);
    return;
  }
  const int within = c % dim;                        // q heads then k heads, both `dim` wide
  if (within >= dims && slot < 0) return;            // passes unchanged and is not cached
  load8<T>(x, f);
  if (within < dims) {
    const float4* cs = reinterpret_cast<const float4*>(table + (int64_t)t * (dims / 2) + within / 2);
    const float4 a = cs[0], b = cs[1];               // (cos, sin) of four neighbouring pairs
    const float co[4] = {a.x, a.z, b.x, b.z}, si[4] = {a.y, a.w, b.y, b.w};
    float r[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      r[2 * i] = f[2 * i] * co[i] - f[2 * i + 1] * si[i];
      r[2 * i + 1] = f[2 * i + 1] * co[i] + f[2 * i] * si[i];
    }
    store8<T>(x, r);
    load8<T>(x, f);
  }
  if (slot >= 0 && c >= nq) store8<T>(k_cache + slot * (int64_t)nk + (c - nq), f);
}

// out[t, h, :] = x[t, h, :] * sigmoid(gate[t, h]): one logit per (token, head). In place when out == x.
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ gate, int64_t gate_stride,
                 int64_t total, int H, int vdim) {
  pdl_wait();
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const int64_t th = e / vdim;
  const int64_t t = th / H;
  const int hd = (int)(th % H);
  out[e] = from_f32<T>(to_f32<T>(x[e]) * sigmoid_f(to_f32<T>(gate[t * gate_stride + hd])));
}

// 16-byte form (vdim % 8 == 0): one thread per 8 consecutive columns, which lie in one head
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_vec_kernel(T* __restrict__ out, const T* __restrict__ x, const T* __restrict__ gate, int64_t gate_stride,
                     int64_t vecs, int H, int vdim) {
  pdl_wait();
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= vecs) return;
  const int64_t th = e * 8 / vdim;
  const float s = sigmoid_f(to_f32<T>(gate[(th / H) * gate_stride + (int)(th % H)]));
  float f[8];
  load8<T>(x + e * 8, f);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] *= s;
  store8<T>(out + e * 8, f);
}

}  // namespace b200

using namespace b200;

extern "C" int b200_residual_rmsnorm(void* out, const float* residual, const float* weight, float offset,
                                     float eps, int32_t rows, int32_t hidden, int32_t dtype,
                                     b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || hidden <= 0, B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!out || !residual || !weight, B200_ERR_NULL_POINTER);
  B200_DISPATCH_3(dtype, T, launch_pdl(residual_rmsnorm_kernel<T>, dim3(rows), dim3(256), 0,
                                       (cudaStream_t)stream, (T*)out, residual, weight, offset, eps, hidden));
  return finish_launch();
}

extern "C" int b200_residual_add_norms(void* h, float* residual, const void* y, const float* w_post,
                                       const float* w_pre, float offset, float eps, int32_t rows,
                                       int32_t hidden, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || hidden <= 0, B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!residual || !y || !w_post || (w_pre && !h), B200_ERR_NULL_POINTER);
  const size_t smem = (size_t)hidden * sizeof(float);
  B200_RETURN_IF(smem > 200 * 1024, B200_ERR_UNSUPPORTED);
  if (hidden % 8 == 0 && hidden <= 8 * 256 * kResVecs && aligned16(residual) && aligned16(y) && aligned16(w_post) &&
      (!w_pre || (aligned16(w_pre) && aligned16(h)))) {
    const int threads = hidden / 8 >= 256 ? 256 : ((hidden / 8 + 31) / 32) * 32;
    B200_DISPATCH_3(dtype, T, launch_pdl(residual_add_norms_vec_kernel<T>, dim3(rows), dim3(threads), 0,
                                         (cudaStream_t)stream, (T*)h, residual, (const T*)y, w_post, w_pre, offset,
                                         eps, hidden));
    return finish_launch();
  }
  B200_DISPATCH_3(dtype, T, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(residual_add_norms_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(residual_add_norms_kernel<T>, dim3(rows), dim3(256), smem, (cudaStream_t)stream, (T*)h,
               residual, (const T*)y, w_post, w_pre, offset, eps, hidden);
  });
  return finish_launch();
}

extern "C" int b200_causal_conv(void* out, int64_t out_stride, const void* x, int64_t x_stride,
                                const float* weight, const float* bias, int32_t act, void* state,
                                const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k,
                                const int32_t* ctx_lens, int32_t num_seqs, int32_t max_q, int32_t channels,
                                int32_t taps, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_seqs < 0 || max_q < 0 || channels <= 0 || taps <= 0, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(taps > kConvMaxTaps || taps - 1 > kConvSeg, B200_ERR_UNSUPPORTED);
  if (num_seqs == 0 || max_q == 0) return B200_OK;
  B200_RETURN_IF(!out || !x || !weight || (cu_q == nullptr) == (ctx_lens == nullptr) || (cu_q && !cu_k) ||
                     (state && !state_slots), B200_ERR_NULL_POINTER);
  B200_RETURN_IF(out == x, B200_ERR_UNSUPPORTED);
  if (channels % 8 == 0 && out_stride % 8 == 0 && x_stride % 8 == 0 && aligned16(out) && aligned16(x) &&
      (!state || aligned16(state)) && taps <= 4) {
    const dim3 vgrid((channels / 8 + 127) / 128, (max_q + kConvSeg - 1) / kConvSeg, num_seqs);
    B200_DISPATCH_3(dtype, T, launch_pdl(causal_conv_vec_kernel<T, 4>, vgrid, dim3(128), 0, (cudaStream_t)stream,
                                         (T*)out, out_stride, (const T*)x, x_stride, weight, bias, act, (T*)state,
                                         state_slots, cu_q, cu_k, ctx_lens, channels, taps));
    return finish_launch();
  }
  const dim3 grid((channels + 127) / 128, (max_q + kConvSeg - 1) / kConvSeg, num_seqs);
  B200_DISPATCH_3(dtype, T, launch_pdl(causal_conv_kernel<T>, grid, dim3(128), 0, (cudaStream_t)stream, (T*)out,
                                       out_stride, (const T*)x, x_stride, weight, bias, act, (T*)state,
                                       state_slots, cu_q, cu_k, ctx_lens, channels, taps));
  return finish_launch();
}

extern "C" int b200_unitnorm_temp_cache(void* qkv, int64_t stride, const int64_t* positions, float eps,
                                        float coef, int32_t every, void* k_cache, void* v_cache,
                                        const int32_t* slots, int32_t slot_pairs, int32_t block_size,
                                        int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads,
                                        int32_t dim, int32_t vdim, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_tokens < 0 || num_heads <= 0 || num_kv_heads <= 0 || dim <= 0 || vdim <= 0 || every <= 0,
                 B200_ERR_BAD_SHAPE);
  if (num_tokens == 0) return B200_OK;
  B200_RETURN_IF(!qkv || !positions || (k_cache == nullptr) != (v_cache == nullptr) || (k_cache && !slots),
                 B200_ERR_NULL_POINTER);
  const int64_t units = (int64_t)num_tokens * (num_heads + 2 * num_kv_heads);
  const int gl = dim / 8;
  if (dim % 8 == 0 && (gl & (gl - 1)) == 0 && gl <= 32 && vdim % 8 == 0 && stride % 8 == 0 && aligned16(qkv) &&
      (!k_cache || (aligned16(k_cache) && aligned16(v_cache)))) {
    const int upw = 32 / gl;
    const dim3 vgrid((unsigned)((units + 8 * upw - 1) / (8 * upw)));
#define B200_UNITNORM_VEC(GLV)                                                                                       \
  B200_DISPATCH_3(dtype, T, launch_pdl(unitnorm_temp_cache_vec_kernel<T, GLV>, vgrid, dim3(256), 0,                  \
                                       (cudaStream_t)stream, (T*)qkv, stride, positions, eps, coef, every,          \
                                       (T*)k_cache, (T*)v_cache, slots, slot_pairs, block_size, num_tokens,         \
                                       num_heads, num_kv_heads, vdim))
    switch (gl) {
      case 1: B200_UNITNORM_VEC(1); break;
      case 2: B200_UNITNORM_VEC(2); break;
      case 4: B200_UNITNORM_VEC(4); break;
      case 8: B200_UNITNORM_VEC(8); break;
      case 16: B200_UNITNORM_VEC(16); break;
      default: B200_UNITNORM_VEC(32); break;
    }
#undef B200_UNITNORM_VEC
    return finish_launch();
  }
  const dim3 grid((unsigned)((units + 7) / 8));
  B200_DISPATCH_3(dtype, T, launch_pdl(unitnorm_temp_cache_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream,
                                       (T*)qkv, stride, positions, eps, coef, every, (T*)k_cache, (T*)v_cache,
                                       slots, slot_pairs, block_size, num_tokens, num_heads, num_kv_heads, dim,
                                       vdim));
  return finish_launch();
}

extern "C" int b200_gated_norm(void* out, const void* y, int32_t y_is_f32, const void* gate,
                               int64_t gate_stride, const float* weight, float eps, int32_t rows, int32_t n,
                               int32_t groups, int32_t gate_first, int32_t gate_act, int32_t dtype,
                               b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || n <= 0 || groups <= 0 || n % groups != 0, B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(gate_act < 0 || gate_act > 2, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(!out || !y || (!gate && gate_act != 2), B200_ERR_NULL_POINTER);
  const dim3 grid(rows, weight ? groups : 1);
  const int g = weight ? groups : 1;
  const int len = n / g;
  if (len % 8 == 0 && len <= 4096 && n % 8 == 0 && gate_stride % 8 == 0 && aligned16(out) && aligned16(y) &&
      (!gate || aligned16(gate)) && (!weight || aligned16(weight))) {
    if (weight && g > 1 && len <= 512) {               // a norm per head: warps, not CTAs, per group
      int gl = 1;
      while (gl * 8 < len && gl < 32) gl <<= 1;
      const int64_t warps = ((int64_t)rows * g + 32 / gl - 1) / (32 / gl);
      const dim3 wgrid((unsigned)((warps + 7) / 8));
      B200_DISPATCH_3(dtype, T, {
        if (y_is_f32)
          launch_pdl(gated_norm_warp_kernel<T, float>, wgrid, dim3(256), 0, (cudaStream_t)stream, (T*)out,
                     (const float*)y, (const T*)gate, gate_stride, weight, eps, (int64_t)rows, n, g, gate_first, gate_act, gl);
        else
          launch_pdl(gated_norm_warp_kernel<T, T>, wgrid, dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)y,
                     (const T*)gate, gate_stride, weight, eps, (int64_t)rows, n, g, gate_first, gate_act, gl);
      });
      return finish_launch();
    }
    const int threads = len / 8 >= 256 ? 256 : ((len / 8 + 31) / 32) * 32;
    B200_DISPATCH_3(dtype, T, {
      if (y_is_f32)
        launch_pdl(gated_norm_vec_kernel<T, float>, grid, dim3(threads), 0, (cudaStream_t)stream, (T*)out,
                   (const float*)y, (const T*)gate, gate_stride, weight, eps, n, g, gate_first, gate_act);
      else
        launch_pdl(gated_norm_vec_kernel<T, T>, grid, dim3(threads), 0, (cudaStream_t)stream, (T*)out, (const T*)y,
                   (const T*)gate, gate_stride, weight, eps, n, g, gate_first, gate_act);
    });
    return finish_launch();
  }
  B200_DISPATCH_3(dtype, T, {
    if (y_is_f32)
      launch_pdl(gated_norm_kernel<T, float>, grid, dim3(256), 0, (cudaStream_t)stream, (T*)out,
                 (const float*)y, (const T*)gate, gate_stride, weight, eps, n, g, gate_first, gate_act);
    else
      launch_pdl(gated_norm_kernel<T, T>, grid, dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)y,
                 (const T*)gate, gate_stride, weight, eps, n, g, gate_first, gate_act);
  });
  return finish_launch();
}

extern "C" int b200_act_and_mul(void* out, const void* x, int32_t rows, int32_t inter, int32_t act,
                                int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || inter <= 0 || act < 0 || act > 2, B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!out || !x, B200_ERR_NULL_POINTER);
  if (inter % 8 == 0 && aligned16(out) && aligned16(x)) {
    const int64_t vecs = (int64_t)rows * (inter / 8);
    int vgrid = (int)((vecs + 255) / 256);
    if (vgrid > 148 * 16) vgrid = 148 * 16;
    B200_DISPATCH_3(dtype, T, launch_pdl(act_and_mul_vec_kernel<T>, dim3(vgrid), dim3(256), 0, (cudaStream_t)stream,
                                         (T*)out, (const T*)x, (int64_t)rows, inter / 8, act));
    return finish_launch();
  }
  const int64_t total = (int64_t)rows * inter;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  B200_DISPATCH_3(dtype, T, launch_pdl(act_and_mul_kernel<T>, dim3(grid), dim3(256), 0, (cudaStream_t)stream,
                                       (T*)out, (const T*)x, (int64_t)rows, inter, act));
  return finish_launch();
}

extern "C" int b200_act_only(void* out, const void* x, int64_t total, int32_t act, int32_t dtype,
                             b200_stream_t stream) {
  B200_RETURN_IF(total < 0 || act < 0 || act > 3, B200_ERR_BAD_SHAPE);
  if (total == 0) return B200_OK;
  B200_RETURN_IF(!out || !x, B200_ERR_NULL_POINTER);
  if (total % 8 == 0 && aligned16(out) && aligned16(x)) {
    int vgrid = (int)((total / 8 + 255) / 256);
    if (vgrid > 148 * 16) vgrid = 148 * 16;
    B200_DISPATCH_3(dtype, T, launch_pdl(act_only_vec_kernel<T>, dim3(vgrid), dim3(256), 0, (cudaStream_t)stream,
                                         (T*)out, (const T*)x, total / 8, act));
    return finish_launch();
  }
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  B200_DISPATCH_3(dtype, T, launch_pdl(act_only_kernel<T>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (T*)out,
                                       (const T*)x, total, act));
  return finish_launch();
}

extern "C" int b200_norm_residual(void* h, float* residual, const void* y, const int64_t* y_index, int64_t y_rows,
                                  const void* y2, const int64_t* y2_index, int64_t y2_rows, const float* w,
                                  const float* b, float eps, float offset, int32_t kind, int32_t accumulate,
                                  int32_t rows, int32_t hidden, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || hidden <= 0 || (kind != 0 && kind != 1), B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!residual || !y || !w, B200_ERR_NULL_POINTER);
  B200_RETURN_IF((y_index && y_rows <= 0) || (y2 && y2_index && y2_rows <= 0), B200_ERR_BAD_SHAPE);
  const size_t smem = (size_t)hidden * sizeof(float);
  B200_RETURN_IF(smem > 200 * 1024, B200_ERR_UNSUPPORTED);
  if (hidden % 8 == 0 && hidden <= 8 * 256 * kResVecs && aligned16(residual) && aligned16(y) && aligned16(w) &&
      (!b || aligned16(b)) && (!y2 || aligned16(y2)) && (!h || aligned16(h))) {
    const int threads = hidden / 8 >= 256 ? 256 : ((hidden / 8 + 31) / 32) * 32;
    B200_DISPATCH_3(dtype, T, launch_pdl(norm_residual_vec_kernel<T>, dim3(rows), dim3(threads), 0,
                                         (cudaStream_t)stream, (T*)h, residual, (const T*)y, y_index, y_rows,
                                         (const T*)y2, y2_index, y2_rows, w, b, eps, offset, kind, accumulate, hidden));
    return finish_launch();
  }
  B200_DISPATCH_3(dtype, T, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(norm_residual_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(norm_residual_kernel<T>, dim3(rows), dim3(256), smem, (cudaStream_t)stream, (T*)h, residual,
               (const T*)y, y_index, y_rows, (const T*)y2, y2_index, y2_rows, w, b, eps, offset, kind, accumulate,
               hidden);
  });
  return finish_launch();
}

extern "C" int b200_rownorm_cache(void* x, int64_t stride, const float* wq, const float* wk, float eps,
                                  void* k_cache, void* v_cache, const int32_t* slots, int32_t slot_pairs,
                                  int32_t block_size, int32_t num_tokens, int32_t nq, int32_t nk, int32_t nv,
                                  int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_tokens < 0 || nq <= 0 || nk < 0 || nv < 0, B200_ERR_BAD_SHAPE);
  if (num_tokens == 0) return B200_OK;
  B200_RETURN_IF(!x || !wq || (nk > 0 && !wk) || (k_cache == nullptr) != (v_cache == nullptr) || (k_cache && !slots),
                 B200_ERR_NULL_POINTER);
  B200_RETURN_IF(k_cache && (nk <= 0 || nv <= 0), B200_ERR_BAD_SHAPE);
  const dim3 grid(num_tokens, nk > 0 ? (k_cache ? 3 : 2) : 1);
  if (nq % 8 == 0 && nk % 8 == 0 && nv % 8 == 0 && stride % 8 == 0 && aligned16(x) && aligned16(wq) &&
      (!wk || aligned16(wk)) && (!k_cache || (aligned16(k_cache) && aligned16(v_cache)))) {
    const int parts = (int)grid.y;
    const int64_t units = (int64_t)num_tokens * parts;
    B200_DISPATCH_3(dtype, T, launch_pdl(rownorm_cache_vec_kernel<T>, dim3((unsigned)((units + 7) / 8)), dim3(256), 0,
                                         (cudaStream_t)stream, (T*)x, stride, wq, wk, eps, (T*)k_cache, (T*)v_cache,
                                         slots, slot_pairs, block_size, num_tokens, parts, nq, nk, nv));
    return finish_launch();
  }
  B200_DISPATCH_3(dtype, T, launch_pdl(rownorm_cache_kernel<T>, grid, dim3(128), 0, (cudaStream_t)stream, (T*)x,
                                       stride, wq, wk, eps, (T*)k_cache, (T*)v_cache, slots, slot_pairs, block_size,
                                       nq, nk, nv));
  return finish_launch();
}

extern "C" int b200_gate_prep(float* q_out, float* f_out, const void* q, int64_t q_stride, const void* f,
                              int64_t f_stride, const float* bias, const float* lower, int32_t num_tokens,
                              int32_t n, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_tokens < 0 || n <= 0, B200_ERR_BAD_SHAPE);
  if (num_tokens == 0) return B200_OK;
  B200_RETURN_IF(!q_out || !f_out || !q || !f, B200_ERR_NULL_POINTER);
  const int64_t total = (int64_t)num_tokens * n;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  B200_DISPATCH_3(dtype, T, launch_pdl(gate_prep_kernel<T>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, q_out,
                                       f_out, (const T*)q, q_stride, (const T*)f, f_stride, bias, lower,
                                       (int64_t)num_tokens, n));
  return finish_launch();
}

extern "C" int b200_gather_rows_by_head(void* out, const void* src, int64_t src_stride_bytes, const int64_t* slots,
                                        int64_t entries, int32_t nk, int32_t num_kv_heads, int32_t head_bytes,
                                        b200_stream_t stream) {
  B200_RETURN_IF(entries < 0 || nk <= 0 || num_kv_heads <= 0 || head_bytes <= 0, B200_ERR_BAD_SHAPE);
  if (entries == 0) return B200_OK;
  B200_RETURN_IF(!out || !src || !slots, B200_ERR_NULL_POINTER);
  B200_RETURN_IF(head_bytes % 16 != 0 || src_stride_bytes % 16 != 0 || !aligned16(out) || !aligned16(src),
                 B200_ERR_MISALIGNED);
  const int vph = head_bytes / 16;
  const int64_t total = entries * nk * num_kv_heads * vph;
  int64_t blocks = (total + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  launch_pdl(gather_rows_by_head_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (uint4*)out,
             (const char*)src, src_stride_bytes, slots, total, nk, num_kv_heads, vph);
  return finish_launch();
}


extern "C" int b200_residual_scale_groupnorm(void* h, float* residual, const void* y, const int64_t* y_index,
                                             int64_t y_rows, const float* scale, float c, int32_t accumulate,
                                             const float* weight, float offset, float eps, int32_t rows,
                                             int32_t hidden, int32_t groups, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || hidden <= 0 || groups <= 0 || hidden % groups != 0 || (y_index && y_rows <= 0),
                 B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!residual || (weight && !h) || (y_index && !y) || (!accumulate && !y), B200_ERR_NULL_POINTER);
  const int per = hidden / groups;
  if (hidden % 8 == 0 && per % 8 == 0 && hidden <= 8 * 256 * kResVecs && groups <= 256 && aligned16(residual) &&
      (!y || aligned16(y)) && (!scale || aligned16(scale)) && (!weight || (aligned16(weight) && aligned16(h)))) {
    const int threads = hidden / 8 >= 256 ? 256 : ((hidden / 8 + 31) / 32) * 32;
    B200_DISPATCH_3(dtype, T, launch_pdl(residual_scale_groupnorm_vec_kernel<T>, dim3(rows), dim3(threads), 0,
                                         (cudaStream_t)stream, (T*)h, residual, (const T*)y, y_index, y_rows, scale,
                                         c, accumulate, weight, offset, eps, hidden, groups));
    return finish_launch();
  }
  const size_t smem = (size_t)(hidden + groups) * sizeof(float);
  B200_RETURN_IF(smem > 200 * 1024, B200_ERR_UNSUPPORTED);
  B200_DISPATCH_3(dtype, T, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(residual_scale_groupnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(residual_scale_groupnorm_kernel<T>, dim3(rows), dim3(256), smem, (cudaStream_t)stream, (T*)h, residual,
               (const T*)y, y_index, y_rows, scale, c, accumulate, weight, offset, eps, hidden, groups);
  });
  return finish_launch();
}

extern "C" int b200_rotary_table(float* table, const int64_t* positions, const double* freq, double magnitude,
                                 int32_t tokens, int32_t half, b200_stream_t stream) {
  B200_RETURN_IF(tokens < 0 || half <= 0, B200_ERR_BAD_SHAPE);
  if (tokens == 0) return B200_OK;
  B200_RETURN_IF(!table || !positions || !freq, B200_ERR_NULL_POINTER);
  const int64_t total = (int64_t)tokens * half;
  launch_pdl(rotary_table_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, (cudaStream_t)stream,
             (float2*)table, positions, freq, magnitude, tokens, half);
  return finish_launch();
}

extern "C" int b200_rope_mix_cache(void* qkv, int64_t stride, const float* table, int32_t dims, int32_t interleaved,
                                   const void* v_other, int64_t v_other_stride, const float* lambda, void* k_cache,
                                   void* v_cache, const int32_t* slots, int32_t slot_pairs, int32_t block_size,
                                   int32_t num_tokens, int32_t num_heads, int32_t num_kv_heads, int32_t dim,
                                   int32_t vdim, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_tokens < 0 || num_heads <= 0 || num_kv_heads <= 0 || dim <= 0 || vdim <= 0 || dims < 0 ||
                     dims > dim || dims % 2 != 0,
                 B200_ERR_BAD_SHAPE);
  if (num_tokens == 0) return B200_OK;
  B200_RETURN_IF(!qkv || (dims > 0 && !table) || (k_cache == nullptr) != (v_cache == nullptr) || (k_cache && !slots) ||
                     (v_other && !lambda),
                 B200_ERR_NULL_POINTER);
  if (interleaved && dim % 8 == 0 && vdim % 8 == 0 && dims % 8 == 0 && stride % 8 == 0 && aligned16(qkv) &&
      (!v_other || (aligned16(v_other) && v_other_stride % 8 == 0)) &&
      (!k_cache || (aligned16(k_cache) && aligned16(v_cache))) && (dims == 0 || aligned16(table))) {
    const int64_t total = (int64_t)num_tokens * ((num_heads * dim + num_kv_heads * (dim + vdim)) / 8);
    B200_DISPATCH_3(dtype, T, launch_pdl(rope_mix_cache_vec_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256),
                                         0, (cudaStream_t)stream, (T*)qkv, stride, (const float2*)table, dims,
                                         (const T*)v_other, v_other_stride, lambda, (T*)k_cache, (T*)v_cache, slots,
                                         slot_pairs, block_size, num_tokens, num_heads, num_kv_heads, dim, vdim));
    return finish_launch();
  }
  const int64_t units = (int64_t)num_tokens * (num_heads + 2 * num_kv_heads);
  const dim3 grid((unsigned)((units + 7) / 8));
  B200_DISPATCH_3(dtype, T, launch_pdl(rope_mix_cache_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, (T*)qkv,
                                       stride, (const float2*)table, dims, interleaved, (const T*)v_other,
                                       v_other_stride, lambda, (T*)k_cache, (T*)v_cache, slots, slot_pairs, block_size,
                                       num_tokens, num_heads, num_kv_heads, dim, vdim));
  return finish_launch();
}

extern "C" int b200_head_gate(void* out, const void* x, const void* gate, int64_t gate_stride, int32_t rows,
                              int32_t num_heads, int32_t vdim, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || num_heads <= 0 || vdim <= 0, B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!out || !x || !gate, B200_ERR_NULL_POINTER);
  const int64_t total = (int64_t)rows * num_heads * vdim;
  if (vdim % 8 == 0 && aligned16(out) && aligned16(x)) {
    B200_DISPATCH_3(dtype, T, launch_pdl(head_gate_vec_kernel<T>, dim3((unsigned)((total / 8 + 255) / 256)), dim3(256), 0,
                                         (cudaStream_t)stream, (T*)out, (const T*)x, (const T*)gate, gate_stride,
                                         total / 8, num_heads, vdim));
    return finish_launch();
  }
  B200_DISPATCH_3(dtype, T, launch_pdl(head_gate_kernel<T>, dim3((unsigned)((total + 255) / 256)), dim3(256), 0,
                                       (cudaStream_t)stream, (T*)out, (const T*)x, (const T*)gate, gate_stride, total,
                                       num_heads, vdim));
  return finish_launch();
}
