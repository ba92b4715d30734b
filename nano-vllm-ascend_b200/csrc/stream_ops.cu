// stream_ops.cu -- row-wise kernels of decoders that keep SEVERAL residual streams (hyper-connections), rotate
// parts of their heads, or feed a recurrence with fp32 unit vectors and per-channel decays:
//
//   stream_mix_norm     x_t <- sum_s mix[s][t] x_s + out[t] y for all streams at once, then u = sum_t in[t] x_t and
//                       h = norm(u): the "residual add + next pre-norm" of a multi-stream residual in ONE launch.
//                       norm is a layer norm with weight and bias, or an RMS norm with a (offset + w) weight.
//   rotary_heads        rotary positions on the first `dims` columns of every head (pairs (2i, 2i+1) or
//                       (i, i + dims/2)), a scale per head range, output in fp32 or the element type, with free
//                       input/output head strides (so that a rotated part can be written into a wider head).
//   delta_prep          what a gated delta rule reads besides v: q and k as fp32 unit vectors (q scaled), the
//                       per-channel decay exp(-exp(A) softplus(a + bias)) and beta = sigmoid(b), all fp32.
//   latent_kv_prep      RMS norm of the query latent; RMS norm of the key/value latent and rotation of the shared
//                       rotated key, written as one cache row [latent | rotated key] (packed and/or paged).
//   glu_clamped         min(g, L) sigmoid(alpha min(g, L)) (clamp(u, -L, L) + 1) for a gated feed-forward.
//   masked_softmax      softmax over the visible keys of a block of fp32 scores (attention composed of library products).
//   mixed_softmax       the same for heads that are mixed BEFORE the softmax: distance bias, [H, H] mix, mask, sink.
//
// All arithmetic is fp32 (angles in fp64: a position times a frequency loses digits in fp32 at long range).
#include "seq_common.cuh"

namespace b200 {

constexpr int kMaxStreams = 8;

struct StreamMixParams {
  float* x;               // [rows, S, hidden] fp32 streams, updated in place
  const void* y;          // [rows, hidden] sublayer output (element type) or nullptr: no update
  const float* mix;       // [S, S] (from, to) or nullptr with y == nullptr
  const float* out_w;     // [S]
  const float* in_w;      // [S] read weights of the NEXT sublayer (nullptr: all ones, the sum of the streams)
  const float* w;         // [hidden] norm weight (nullptr: no h is produced)
  const float* b;         // [hidden] norm bias (layer norm) or nullptr
  void* h;                // [rows, hidden] element type
  float* sum_out;         // optional [rows, hidden] fp32: u itself (before the norm)
  float eps, offset;
  int S, hidden, kind;    // kind 0: layer norm (w, b); 1: RMS norm, weight offset + w
};

template <typename T>
__global__ void __launch_bounds__(256)
stream_mix_norm_kernel(const StreamMixParams P) {
  extern __shared__ float su[];                       // [hidden]
  __shared__ float red[32];
  __shared__ float smix[kMaxStreams * kMaxStreams], sout[kMaxStreams], sin_[kMaxStreams];
  pdl_wait();
  const int S = P.S, hidden = P.hidden;
  if (threadIdx.x < S * S) smix[threadIdx.x] = P.mix != nullptr ? P.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < S) {
    sout[threadIdx.x] = P.out_w != nullptr ? P.out_w[threadIdx.x] : 0.f;
    sin_[threadIdx.x] = P.in_w != nullptr ? P.in_w[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float* xr = P.x + (int64_t)blockIdx.x * S * hidden;
  const T* yr = P.y != nullptr ? (const T*)P.y + (int64_t)blockIdx.x * hidden : nullptr;
  float part = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float xs[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) xs[s] = s < S ? xr[(int64_t)s * hidden + i] : 0.f;
    float u = 0.f;
    if (yr != nullptr) {
      const float y = to_f32<T>(yr[i]);
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t < S) {
          float acc = 0.f;
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < S) acc += smix[s * S + t] * xs[s];
          acc += sout[t] * y;
          xr[(int64_t)t * hidden + i] = acc;
          u += sin_[t] * acc;
        }
      }
    } else {
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t)
        if (t < S) u += sin_[t] * xs[t];
    }
    su[i] = u;
    part += P.kind == 0 ? u : u * u;
  }
  if (P.sum_out != nullptr)
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) P.sum_out[(int64_t)blockIdx.x * hidden + i] = su[i];
  if (P.w == nullptr) return;
  T* h = (T*)P.h + (int64_t)blockIdx.x * hidden;
  if (P.kind == 0) {
    const float mean = cta_sum(part, red) / (float)hidden;
    float sq = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = su[i] - mean;
      sq += d * d;
    }
    const float rstd = 1.0f / sqrtf(cta_sum(sq, red) / (float)hidden + P.eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      h[i] = from_f32<T>((su[i] - mean) * rstd * P.w[i] + (P.b != nullptr ? P.b[i] : 0.f));
  } else {
    const float rstd = 1.0f / sqrtf(cta_sum(part, red) / (float)hidden + P.eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) h[i] = from_f32<T>(su[i] * rstd * (P.offset + P.w[i]));
  }
}

// The same with the stream count as a template parameter and 4 elements per thread and step (hidden % 4 == 0): the
// streams move as 16-byte vectors and the mixing loops are fully unrolled without predicates.
template <typename T, int kS>
__global__ void __launch_bounds__(256)
stream_mix_norm_vec_kernel(const StreamMixParams P) {
  extern __shared__ __align__(16) float su[];         // [hidden]
  __shared__ float red[32];
  __shared__ float smix[kS * kS], sout[kS], sin_[kS];
  pdl_wait();
  const int hidden = P.hidden, nv = hidden / 4;
  if (threadIdx.x < kS * kS) smix[threadIdx.x] = P.mix != nullptr ? P.mix[threadIdx.x] : 0.f;
  if (threadIdx.x < kS) {
    sout[threadIdx.x] = P.out_w != nullptr ? P.out_w[threadIdx.x] : 0.f;
    sin_[threadIdx.x] = P.in_w != nullptr ? P.in_w[threadIdx.x] : 1.f;
  }
  __syncthreads();
  float4* xr = reinterpret_cast<float4*>(P.x + (int64_t)blockIdx.x * kS * hidden);
  const T* yr = P.y != nullptr ? (const T*)P.y + (int64_t)blockIdx.x * hidden : nullptr;
  float part = 0.f;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float xs[kS][4];
#pragma unroll
    for (int s = 0; s < kS; ++s) {
      const float4 v = xr[(int64_t)s * nv + i];
      xs[s][0] = v.x, xs[s][1] = v.y, xs[s][2] = v.z, xs[s][3] = v.w;
    }
    float u[4] = {0.f, 0.f, 0.f, 0.f};
    if (yr != nullptr) {
      float y[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] = to_f32<T>(yr[i * 4 + e]);
#pragma unroll
      for (int t = 0; t < kS; ++t) {
        float acc[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          acc[e] = 0.f;
#pragma unroll
          for (int s = 0; s < kS; ++s) acc[e] += smix[s * kS + t] * xs[s][e];
          acc[e] += sout[t] * y[e];
          u[e] += sin_[t] * acc[e];
        }
        xr[(int64_t)t * nv + i] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      }
    } else {
#pragma unroll
      for (int t = 0; t < kS; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) u[e] += sin_[t] * xs[t][e];
    }
    reinterpret_cast<float4*>(su)[i] = make_float4(u[0], u[1], u[2], u[3]);
#pragma unroll
    for (int e = 0; e < 4; ++e) part += P.kind == 0 ? u[e] : u[e] * u[e];
  }
  if (P.sum_out != nullptr)
    for (int i = threadIdx.x; i < nv; i += blockDim.x)
      reinterpret_cast<float4*>(P.sum_out + (int64_t)blockIdx.x * hidden)[i] = reinterpret_cast<float4*>(su)[i];
  if (P.w == nullptr) return;
  T* h = (T*)P.h + (int64_t)blockIdx.x * hidden;
  float mean = 0.f, rstd;
  if (P.kind == 0) {
    mean = cta_sum(part, red) / (float)hidden;
    float sq = 0.f;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const float4 v = reinterpret_cast<float4*>(su)[i];
      sq += (v.x - mean) * (v.x - mean) + (v.y - mean) * (v.y - mean) + (v.z - mean) * (v.z - mean) +
            (v.w - mean) * (v.w - mean);
    }
    rstd = 1.0f / sqrtf(cta_sum(sq, red) / (float)hidden + P.eps);
  } else {
    rstd = 1.0f / sqrtf(cta_sum(part, red) / (float)hidden + P.eps);
  }
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    const float4 v = reinterpret_cast<float4*>(su)[i];
    const float4 w = reinterpret_cast<const float4*>(P.w)[i];
    const float uu[4] = {v.x, v.y, v.z, v.w}, ww[4] = {w.x, w.y, w.z, w.w};
    float bb[4] = {0.f, 0.f, 0.f, 0.f};
    if (P.kind == 0 && P.b != nullptr) {
      const float4 b = reinterpret_cast<const float4*>(P.b)[i];
      bb[0] = b.x, bb[1] = b.y, bb[2] = b.z, bb[3] = b.w;
    }
#pragma unroll
    for (int e = 0; e < 4; ++e)
      h[i * 4 + e] = from_f32<T>(P.kind == 0 ? (uu[e] - mean) * rstd * ww[e] + bb[e] : uu[e] * rstd * (P.offset + ww[e]));
  }
}

// ------------------------------------------------------------------ rotary positions
struct RotaryParams {
  const void* in;          // element type; head hd of token t starts at in + t * in_stride + hd * in_head
  void* out;               // fp32 or element type; head hd of token t at out + t * out_stride + hd * out_head
  int64_t in_stride, out_stride;
  int in_head, out_head;
  const int64_t* positions;
  int tokens, heads, width, dims, interleaved, split, out_f32;
  int hsplit;                 // threads per (token, pair): each takes every hsplit-th head (few tokens: more threads)
  float scale_lo, scale_hi;   // heads < split are multiplied by scale_lo, the others by scale_hi
  double log2_base;
};

template <typename T>
__global__ void __launch_bounds__(256)
rotary_heads_kernel(const RotaryParams P) {
  pdl_wait();
  const int half = P.dims / 2;
  const int per_tok = half + (P.width - P.dims);      // work items per token: pairs, then pass-through columns
  const int64_t total = (int64_t)P.tokens * per_tok * P.hsplit;
  for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (int64_t)gridDim.x * blockDim.x) {
    const int h0 = (int)(e % P.hsplit);
    const int64_t item = e / P.hsplit;
    const int t = (int)(item / per_tok), w = (int)(item % per_tok);
    const T* src = (const T*)P.in + (int64_t)t * P.in_stride;
    float* of = (float*)P.out + (int64_t)t * P.out_stride;
    T* ot = (T*)P.out + (int64_t)t * P.out_stride;
    if (w < half) {
      const double f = exp2(-(2.0 * (double)w / (double)P.dims) * P.log2_base);
      double sn, cs;
      sincos((double)P.positions[t] * f, &sn, &cs);
      const float c = (float)cs, s = (float)sn;
      const int a = P.interleaved ? 2 * w : w, b = P.interleaved ? 2 * w + 1 : w + half;
      for (int hd = h0; hd < P.heads; hd += P.hsplit) {
        const float sc = hd < P.split ? P.scale_lo : P.scale_hi;
        const float u = to_f32<T>(src[(int64_t)hd * P.in_head + a]), v = to_f32<T>(src[(int64_t)hd * P.in_head + b]);
        const float ra = (u * c - v * s) * sc, rb = (v * c + u * s) * sc;
        if (P.out_f32) {
          of[(int64_t)hd * P.out_head + a] = ra;
          of[(int64_t)hd * P.out_head + b] = rb;
        } else {
          ot[(int64_t)hd * P.out_head + a] = from_f32<T>(ra);
          ot[(int64_t)hd * P.out_head + b] = from_f32<T>(rb);
        }
      }
    } else {
      const int col = P.dims + (w - half);
      for (int hd = h0; hd < P.heads; hd += P.hsplit) {
        const float sc = hd < P.split ? P.scale_lo : P.scale_hi;
        const float u = to_f32<T>(src[(int64_t)hd * P.in_head + col]) * sc;
        if (P.out_f32) of[(int64_t)hd * P.out_head + col] = u;
        else ot[(int64_t)hd * P.out_head + col] = from_f32<T>(u);
      }
    }
  }
}

// ------------------------------------------------------------------ inputs of a gated delta rule
// One warp per (token, unit): units 0 .. 2G-1 are the q and k heads (unit vectors), units 2G .. 2G+H-1 the decay
// rows of the heads (and beta).
template <typename T>
__global__ void __launch_bounds__(256)
delta_prep_kernel(float* __restrict__ qk, float* __restrict__ decay, float* __restrict__ beta,
                  const T* __restrict__ qk_in, int64_t qk_stride, const T* __restrict__ a, int64_t a_stride,
                  const T* __restrict__ b, int64_t b_stride, const float* __restrict__ dt_bias,
                  const float* __restrict__ a_log, int tokens, int H, int G, int dim, float unit_eps, float q_scale) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t unit = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int per_tok = 2 * G + H;
  if (unit >= (int64_t)tokens * per_tok) return;
  const int t = (int)(unit / per_tok), u = (int)(unit % per_tok);
  if (u < 2 * G) {
    const T* x = qk_in + (int64_t)t * qk_stride + (int64_t)u * dim;
    float ss = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float v = to_f32<T>(x[i]);
      ss += v * v;
    }
    const float mul = (u < G ? q_scale : 1.0f) / sqrtf(warp_sum(ss) + unit_eps);
    float* o = qk + (int64_t)t * (2 * G * dim) + (int64_t)u * dim;
    for (int i = lane; i < dim; i += 32) o[i] = to_f32<T>(x[i]) * mul;
    return;
  }
  const int h = u - 2 * G;
  const float rate = expf(a_log[h]);
  const T* ar = a + (int64_t)t * a_stride + (int64_t)h * dim;
  float* o = decay + (int64_t)t * ((int64_t)H * dim) + (int64_t)h * dim;
  for (int i = lane; i < dim; i += 32)
    o[i] = expf(-rate * softplus_f(to_f32<T>(ar[i]) + dt_bias[(int64_t)h * dim + i]));
  if (lane == 0) beta[(int64_t)t * H + h] = sigmoid_f(to_f32<T>(b[(int64_t)t * b_stride + h]));
}

// ------------------------------------------------------------------ latents of a latent attention
// One CTA per token. cq = rms(dq) * wq (element type); row = [rms(c) * wc | rotate(kr)] (element type) into `kc`
// (packed, [tokens, rank + rot]) and, when slots are given, into the paged cache row of the token.
template <typename T>
__global__ void __launch_bounds__(128)
latent_kv_prep_kernel(T* __restrict__ cq, T* __restrict__ kc, T* __restrict__ cache, const int* __restrict__ slots,
                      int slot_pairs, int block_size, const T* __restrict__ dq, int64_t dq_stride,
                      const T* __restrict__ dkv, int64_t dkv_stride, const float* __restrict__ wq,
                      const float* __restrict__ wc, const int64_t* __restrict__ positions, int q_rank, int rank,
                      int rot, int dims, int interleaved, double log2_base, float eps) {
  __shared__ float red[32];
  pdl_wait();
  const int64_t t = blockIdx.x;
  const T* q = dq + t * dq_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = to_f32<T>(q[i]);
    ss += v * v;
  }
  float rstd = 1.0f / sqrtf(cta_sum(ss, red) / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    cq[t * q_rank + i] = from_f32<T>(to_f32<T>(q[i]) * rstd * wq[i]);

  const T* c = dkv + t * dkv_stride;
  ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f32<T>(c[i]);
    ss += v * v;
  }
  rstd = 1.0f / sqrtf(cta_sum(ss, red) / (float)rank + eps);
  const int row = rank + rot;
  T* dst = nullptr;
  if (cache != nullptr) {
    const int64_t slot = slot_pairs ? (int64_t)slots[2 * t] * block_size + slots[2 * t + 1] : (int64_t)slots[t];
    if (slot >= 0) dst = cache + slot * row;
  }
  T* pk = kc != nullptr ? kc + t * row : nullptr;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const T v = from_f32<T>(to_f32<T>(c[i]) * rstd * wc[i]);
    if (pk != nullptr) pk[i] = v;
    if (dst != nullptr) dst[i] = v;
  }
  const int half = dims / 2;
  for (int w = threadIdx.x; w < half + (rot - dims); w += blockDim.x) {
    if (w < half) {
      const double f = exp2(-(2.0 * (double)w / (double)dims) * log2_base);
      double sn, cs;
      sincos((double)positions[t] * f, &sn, &cs);
      const float cc = (float)cs, s = (float)sn;
      const int a = interleaved ? 2 * w : w, b = interleaved ? 2 * w + 1 : w + half;
      const float u = to_f32<T>(c[rank + a]), v = to_f32<T>(c[rank + b]);
      const T ra = from_f32<T>(u * cc - v * s), rb = from_f32<T>(v * cc + u * s);
      if (pk != nullptr) pk[rank + a] = ra, pk[rank + b] = rb;
      if (dst != nullptr) dst[rank + a] = ra, dst[rank + b] = rb;
    } else {
      const int col = dims + (w - half);
      if (pk != nullptr) pk[rank + col] = c[rank + col];
      if (dst != nullptr) dst[rank + col] = c[rank + col];
    }
  }
}

// ------------------------------------------------------------------ clamped gated unit
template <typename T>
__global__ void __launch_bounds__(256)
glu_clamped_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int inter, float alpha, float limit) {
  pdl_wait();
  const int64_t total = rows * inter;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / inter;
    const int c = (int)(i - r * inter);
    const float g = fminf(to_f32<T>(x[r * 2 * inter + c]), limit);
    const float u = fminf(fmaxf(to_f32<T>(x[r * 2 * inter + inter + c]), -limit), limit);
    out[i] = from_f32<T>(g * sigmoid_f(alpha * g) * (u + 1.0f));
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
glu_clamped_vec_kernel(T* __restrict__ out, const T* __restrict__ x, int64_t rows, int inter8, float alpha,
                       float limit) {
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
      const float gg = fminf(g[e], limit), uu = fminf(fmaxf(u[e], -limit), limit);
      o[e] = gg * sigmoid_f(alpha * gg) * (uu + 1.0f);
    }
    store8<T>(out + i * 8, o);
  }
}

// ------------------------------------------------------------------ masked softmax over a block of scores
// One warp per row of s [rows, nk] (fp32 scores of `heads` query heads per token against nk keys). Two forms:
//   ctx_lens == nullptr: the rows are consecutive tokens of ONE sequence, row r at position first_pos + r / heads,
//                        column j is the key at position key_lo + j;
//   ctx_lens != nullptr: row r belongs to sequence r / heads, whose one token sits at position ctx_lens[.] - 1 (0 keys:
//                        a padded row, all zeros), and column j is the key at position pos - nk + 1 + j (the last nk
//                        positions, gathered by the caller; negative positions do not exist).
//   chunk_first != nullptr: the rows come in chunks of rows_per_chunk; chunk c holds consecutive tokens of one sequence
//                        from position chunk_first[c] on, against keys from position chunk_lo[c] on (may be negative).
// A key at position kp is visible iff 0 <= kp <= pos and (window == 0 or kp > pos - window). p = softmax(scale * s)
// over the visible keys, written in the element type; hidden keys get 0.
template <typename T>
__global__ void __launch_bounds__(128)
masked_softmax_kernel(T* __restrict__ p, const float* __restrict__ s, int64_t rows, int nk, int heads, int first_pos,
                      int key_lo, int window, float scale, const int* __restrict__ ctx_lens,
                      const int* __restrict__ chunk_first, const int* __restrict__ chunk_lo, int rows_per_chunk) {
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  int pos = first_pos + (int)(r / heads);
  if (chunk_first != nullptr) {
    const int64_t c = r / rows_per_chunk;
    pos = chunk_first[c] + (int)((r % rows_per_chunk) / heads);
    key_lo = chunk_lo[c];
  } else if (ctx_lens != nullptr) {
    pos = ctx_lens[r / heads] - 1;
    key_lo = pos - nk + 1;
  }
  const int hi = pos < 0 ? 0 : min(nk, pos - key_lo + 1);                    // visible: [lo, hi)
  int lo = max(0, -key_lo);
  if (window > 0) lo = max(lo, pos - window + 1 - key_lo);
  const float* sr = s + r * nk;
  T* pr = p + r * nk;
  float m = -INFINITY;
  for (int j = lo + lane; j < hi; j += 32) m = fmaxf(m, sr[j]);
  m = warp_max(m);
  float l = 0.f;
  for (int j = lo + lane; j < hi; j += 32) l += expf((sr[j] - m) * scale);
  l = warp_sum(l);
  const float inv = l > 0.f ? 1.0f / l : 0.f;
  for (int j = lane; j < nk; j += 32)
    pr[j] = from_f32<T>((j >= lo && j < hi) ? expf((sr[j] - m) * scale) * inv : 0.f);
}

// ------------------------------------------------------------------ softmax of heads that talk to each other
// s: raw dot products fp32 [B, G, C, rep, nk] -- entry b (a chunk of a prompt, or a sequence of a decode step), kv head
// g, token c of the entry, query head g * rep + r, key column j. One CTA per (b, c) holds the token's H x visible-keys
// block in shared memory: x_h(j) = scale s_h(j) - slope_h (pos - key(j)); x'_h = sum_g talk[h][g] x_g; p_h = exp(x'_h) /
// (sum_visible exp(x'_h) + exp(sink_h)), written in the element type over ALL nk columns (hidden keys 0). Positions as
// in masked_softmax: chunks (chunk_first / chunk_lo per entry, token c at chunk_first + c) or one token per sequence
// (ctx_lens; C == 1; the columns are the last nk positions). HM >= H bounds the per-thread column of heads.
template <typename T, int HM>
__global__ void __launch_bounds__(256)
mixed_softmax_kernel(T* __restrict__ p, const float* __restrict__ s, int C, int G, int rep, int nk, int ns, float scale,
                     int window, const float* __restrict__ slopes, const float* __restrict__ talk,
                     const float* __restrict__ sink, const int* __restrict__ ctx_lens,
                     const int* __restrict__ chunk_first, const int* __restrict__ chunk_lo) {
  extern __shared__ __align__(16) float smem_all[];   // talk [H][HM] (columns past H are zero), then x [H][ns]
  pdl_wait();
  const int H = G * rep;
  const int b = blockIdx.y, c = blockIdx.x;
  float* stalk = smem_all;
  float* sm = smem_all + (size_t)H * HM;              // ns >= the most keys any token sees (the window, or nk)
  int pos, key_lo;
  if (chunk_first != nullptr) {
    pos = chunk_first[b] + c;
    key_lo = chunk_lo[b];
  } else {
    pos = ctx_lens[b] - 1;
    key_lo = pos - nk + 1;
  }
  const int hi = pos < 0 ? 0 : min(nk, pos - key_lo + 1);                    // visible: columns [lo, hi)
  int lo = max(0, -key_lo);
  if (window > 0) lo = max(lo, pos - window + 1 - key_lo);
  const int nv = max(0, hi - lo);
  if (talk != nullptr)
    for (int e = threadIdx.x; e < H * HM; e += blockDim.x) stalk[e] = e % HM < H ? talk[(e / HM) * H + e % HM] : 0.f;
  const int64_t row0 = ((int64_t)b * G * C + c) * rep;                       // row of head (g, r): row0 + g C rep + r
  const int64_t gstep = (int64_t)C * rep;
  // every thread keeps several loads in flight: one pass over (head, key) pairs, four heads per step
  for (int h0 = 0; h0 < H; h0 += 4) {
    for (int j = threadIdx.x; j < nv; j += blockDim.x) {
      float raw[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int h = h0 + u;
        raw[u] = h < H ? s[(row0 + (h / rep) * gstep + h % rep) * nk + lo + j] : 0.f;
      }
      const float dist = (float)(pos - (key_lo + lo + j));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int h = h0 + u;
        if (h < H) sm[(size_t)h * ns + j] = raw[u] * scale - (slopes != nullptr ? slopes[h] : 0.f) * dist;
      }
    }
  }
  __syncthreads();
  if (talk != nullptr) {
    for (int j = threadIdx.x; j < nv; j += blockDim.x) {                     // a thread mixes one key's column of heads
      float v[HM];
#pragma unroll
      for (int g = 0; g < HM; ++g) v[g] = g < H ? sm[(size_t)g * ns + j] : 0.f;
      for (int h = 0; h < H; ++h) {
        const float4* tr = reinterpret_cast<const float4*>(stalk + h * HM);     // one broadcast load per four heads
        float d0 = 0.f, d1 = 0.f;
#pragma unroll
        for (int g = 0; g < HM / 4; ++g) {
          const float4 t4 = tr[g];
          d0 += t4.x * v[4 * g] + t4.z * v[4 * g + 2];
          d1 += t4.y * v[4 * g + 1] + t4.w * v[4 * g + 3];
        }
        sm[(size_t)h * ns + j] = d0 + d1;
      }
    }
    __syncthreads();
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int h = warp; h < H; h += nw) {
    float* x = sm + (size_t)h * ns;
    float m = -INFINITY;
    for (int j = lane; j < nv; j += 32) m = fmaxf(m, x[j]);
    m = warp_max(m);
    const float sk = sink != nullptr ? sink[h] : -INFINITY;
    m = fmaxf(m, sk);
    float l = 0.f;
    for (int j = lane; j < nv; j += 32) {
      const float e = expf(x[j] - m);
      x[j] = e;
      l += e;
    }
    l = warp_sum(l) + (sink != nullptr ? expf(sk - m) : 0.f);
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* pr = p + (row0 + (h / rep) * gstep + h % rep) * nk;
    for (int j = lane; j < nk; j += 32) pr[j] = from_f32<T>((j >= lo && j < hi) ? x[j - lo] * inv : 0.f);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_mixed_softmax(void* p, const float* s, int32_t entries, int32_t tokens_per_entry,
                                  int32_t num_kv_heads, int32_t rep, int32_t nk, float scale, int32_t window,
                                  const float* slopes, const float* talk, const float* sink,
                                  const int32_t* ctx_lens, const int32_t* chunk_first, const int32_t* chunk_lo,
                                  int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(entries < 0 || tokens_per_entry <= 0 || num_kv_heads <= 0 || rep <= 0 || nk <= 0 || window < 0,
                 B200_ERR_BAD_SHAPE);
  if (entries == 0) return B200_OK;
  B200_RETURN_IF(!p || !s || (ctx_lens == nullptr) == (chunk_first == nullptr) || (chunk_first && !chunk_lo),
                 B200_ERR_NULL_POINTER);
  B200_RETURN_IF(ctx_lens && tokens_per_entry != 1, B200_ERR_BAD_SHAPE);
  const int H = num_kv_heads * rep;
  B200_RETURN_IF(H > 64 || entries > 65535, B200_ERR_UNSUPPORTED);
  const int hm = H <= 4 ? 4 : H <= 8 ? 8 : H <= 16 ? 16 : H <= 32 ? 32 : 64;
  const int ns = window > 0 && window < nk ? window : nk;          // no token sees more keys than its window holds
  const size_t smem = ((size_t)H * ns + (size_t)H * hm) * sizeof(float);
  B200_RETURN_IF(smem > 200 * 1024, B200_ERR_UNSUPPORTED);
  const dim3 grid(tokens_per_entry, entries);
#define B200_MIXSM(HMV)                                                                                              \
  B200_DISPATCH_3(dtype, T, {                                                                                        \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(mixed_softmax_kernel<T, HMV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
    launch_pdl(mixed_softmax_kernel<T, HMV>, grid, dim3(256), smem, (cudaStream_t)stream, (T*)p, s,                  \
               tokens_per_entry, num_kv_heads, rep, nk, ns, scale, window, slopes, talk, sink, ctx_lens,             \
               chunk_first, chunk_lo);                                                                               \
  })
  if (H <= 4) B200_MIXSM(4);
  else if (H <= 8) B200_MIXSM(8);
  else if (H <= 16) B200_MIXSM(16);
  else if (H <= 32) B200_MIXSM(32);
  else B200_MIXSM(64);
#undef B200_MIXSM
  return finish_launch();
}

extern "C" int b200_masked_softmax(void* p, const float* s, int64_t rows, int32_t nk, int32_t heads,
                                   int32_t first_pos, int32_t key_lo, int32_t window, float scale,
                                   const int32_t* ctx_lens, const int32_t* chunk_first, const int32_t* chunk_lo,
                                   int32_t rows_per_chunk, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || nk <= 0 || heads <= 0 || first_pos < 0 || window < 0 || scale <= 0.f,
                 B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!p || !s || (chunk_first && (!chunk_lo || rows_per_chunk <= 0)), B200_ERR_NULL_POINTER);
  B200_DISPATCH_3(dtype, T, launch_pdl(masked_softmax_kernel<T>, dim3((unsigned)((rows + 3) / 4)), dim3(128), 0,
                                       (cudaStream_t)stream, (T*)p, s, rows, nk, heads, first_pos, key_lo, window,
                                       scale, ctx_lens, chunk_first, chunk_lo, rows_per_chunk));
  return finish_launch();
}

extern "C" int b200_stream_mix_norm(void* h, float* x, const void* y, const float* mix, const float* out_w,
                                    const float* in_w, const float* w, const float* b, float* sum_out,
                                    float eps, float offset, int32_t kind, int32_t rows, int32_t streams,
                                    int32_t hidden, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || streams <= 0 || hidden <= 0 || (kind != 0 && kind != 1), B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(streams > kMaxStreams || hidden > 48 * 1024, B200_ERR_UNSUPPORTED);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!x || (y && (!mix || !out_w)) || (w && !h), B200_ERR_NULL_POINTER);
  StreamMixParams P;
  P.x = x, P.y = y, P.mix = mix, P.out_w = out_w, P.in_w = in_w, P.w = w, P.b = b, P.h = h, P.sum_out = sum_out;
  P.eps = eps, P.offset = offset, P.S = streams, P.hidden = hidden, P.kind = kind;
  const size_t smem = (size_t)hidden * sizeof(float);
  const bool vec = hidden % 4 == 0 && smem <= 40 * 1024 && aligned16(x) && (!w || aligned16(w)) &&
                   (!b || aligned16(b)) && (!sum_out || aligned16(sum_out));
#define B200_STREAMS_VEC(N)                                                                                        \
  case N:                                                                                                          \
    B200_DISPATCH_3(dtype, T, launch_pdl(stream_mix_norm_vec_kernel<T, N>, dim3(rows), dim3(256), smem,            \
                                         (cudaStream_t)stream, P));                                                \
    return finish_launch();
  if (vec) {
    switch (streams) {
      B200_STREAMS_VEC(1)
      B200_STREAMS_VEC(2)
      B200_STREAMS_VEC(3)
      B200_STREAMS_VEC(4)
      B200_STREAMS_VEC(5)
      B200_STREAMS_VEC(6)
      B200_STREAMS_VEC(7)
      B200_STREAMS_VEC(8)
    }
  }
#undef B200_STREAMS_VEC
  B200_DISPATCH_3(dtype, T, {
    if (smem > 40 * 1024)
      cudaFuncSetAttribute(stream_mix_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(stream_mix_norm_kernel<T>, dim3(rows), dim3(256), smem, (cudaStream_t)stream, P);
  });
  return finish_launch();
}

extern "C" int b200_rotary_heads(void* out, int64_t out_stride, int32_t out_head, int32_t out_f32, const void* in,
                                 int64_t in_stride, int32_t in_head, const int64_t* positions, int32_t tokens,
                                 int32_t heads, int32_t width, int32_t dims, double base, int32_t interleaved,
                                 int32_t split, float scale_lo, float scale_hi, int32_t dtype,
                                 b200_stream_t stream) {
  B200_RETURN_IF(tokens < 0 || heads <= 0 || width <= 0 || dims < 0 || dims > width || dims % 2 != 0 || base <= 0.0,
                 B200_ERR_BAD_SHAPE);
  if (tokens == 0) return B200_OK;
  B200_RETURN_IF(!out || !in || !positions, B200_ERR_NULL_POINTER);
  RotaryParams P;
  P.in = in, P.out = out, P.in_stride = in_stride, P.out_stride = out_stride, P.in_head = in_head;
  P.out_head = out_head, P.positions = positions, P.tokens = tokens, P.heads = heads, P.width = width;
  P.dims = dims, P.interleaved = interleaved, P.split = split, P.out_f32 = out_f32, P.scale_lo = scale_lo;
  P.scale_hi = scale_hi, P.log2_base = log2(base);
  const int64_t items = (int64_t)tokens * (dims / 2 + (width - dims));
  int64_t hsplit = items > 0 ? 32768 / items : 1;     // a decode step has few (token, pair) items: split the heads too
  if (hsplit < 1) hsplit = 1;
  if (hsplit > heads) hsplit = heads;
  P.hsplit = (int)hsplit;
  const int64_t total = items * hsplit;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  B200_DISPATCH_3(dtype, T, launch_pdl(rotary_heads_kernel<T>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, P));
  return finish_launch();
}

extern "C" int b200_delta_prep(float* qk, float* decay, float* beta, const void* qk_in, int64_t qk_stride,
                               const void* a, int64_t a_stride, const void* b, int64_t b_stride,
                               const float* dt_bias, const float* a_log, int32_t tokens, int32_t num_heads,
                               int32_t groups, int32_t dim, float unit_eps, float q_scale, int32_t dtype,
                               b200_stream_t stream) {
  B200_RETURN_IF(tokens < 0 || num_heads <= 0 || groups <= 0 || dim <= 0, B200_ERR_BAD_SHAPE);
  if (tokens == 0) return B200_OK;
  B200_RETURN_IF(!qk || !decay || !beta || !qk_in || !a || !b || !dt_bias || !a_log, B200_ERR_NULL_POINTER);
  const int64_t units = (int64_t)tokens * (2 * groups + num_heads);
  const dim3 grid((unsigned)((units + 7) / 8));
  B200_DISPATCH_3(dtype, T, launch_pdl(delta_prep_kernel<T>, grid, dim3(256), 0, (cudaStream_t)stream, qk, decay, beta,
                                       (const T*)qk_in, qk_stride, (const T*)a, a_stride, (const T*)b, b_stride,
                                       dt_bias, a_log, tokens, num_heads, groups, dim, unit_eps, q_scale));
  return finish_launch();
}

extern "C" int b200_latent_kv_prep(void* cq, void* kc, void* cache, const int32_t* slots, int32_t slot_pairs,
                                   int32_t block_size, const void* dq, int64_t dq_stride, const void* dkv,
                                   int64_t dkv_stride, const float* wq, const float* wc, const int64_t* positions,
                                   int32_t tokens, int32_t q_rank, int32_t rank, int32_t rot, int32_t dims,
                                   double base, int32_t interleaved, float eps, int32_t dtype,
                                   b200_stream_t stream) {
  B200_RETURN_IF(tokens < 0 || q_rank <= 0 || rank <= 0 || rot < 0 || dims < 0 || dims > rot || dims % 2 != 0 ||
                     base <= 0.0, B200_ERR_BAD_SHAPE);
  if (tokens == 0) return B200_OK;
  B200_RETURN_IF(!cq || !dq || !dkv || !wq || !wc || !positions || (cache && !slots), B200_ERR_NULL_POINTER);
  B200_DISPATCH_3(dtype, T, launch_pdl(latent_kv_prep_kernel<T>, dim3(tokens), dim3(128), 0, (cudaStream_t)stream,
                                       (T*)cq, (T*)kc, (T*)cache, slots, slot_pairs, block_size, (const T*)dq,
                                       dq_stride, (const T*)dkv, dkv_stride, wq, wc, positions, q_rank, rank, rot,
                                       dims, interleaved, log2(base), eps));
  return finish_launch();
}

extern "C" int b200_glu_clamped(void* out, const void* x, int32_t rows, int32_t inter, float alpha, float limit,
                                int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(rows < 0 || inter <= 0, B200_ERR_BAD_SHAPE);
  if (rows == 0) return B200_OK;
  B200_RETURN_IF(!out || !x, B200_ERR_NULL_POINTER);
  if (inter % 8 == 0 && aligned16(out) && aligned16(x)) {
    const int64_t vecs = (int64_t)rows * (inter / 8);
    int vgrid = (int)((vecs + 255) / 256);
    if (vgrid > 148 * 16) vgrid = 148 * 16;
    B200_DISPATCH_3(dtype, T, launch_pdl(glu_clamped_vec_kernel<T>, dim3(vgrid), dim3(256), 0, (cudaStream_t)stream,
                                         (T*)out, (const T*)x, (int64_t)rows, inter / 8, alpha, limit));
    return finish_launch();
  }
  const int64_t total = (int64_t)rows * inter;
  int grid = (int)((total + 255) / 256);
  if (grid > 148 * 16) grid = 148 * 16;
  B200_DISPATCH_3(dtype, T, launch_pdl(glu_clamped_kernel<T>, dim3(grid), dim3(256), 0, (cudaStream_t)stream, (T*)out,
                                       (const T*)x, (int64_t)rows, inter, alpha, limit));
  return finish_launch();
}
