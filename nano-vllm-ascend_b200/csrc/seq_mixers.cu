// seq_mixers.cu -- the two sequence mixers that the tcgen05 attention kernels do not cover:
//
//   attn_generic       causal softmax attention for ANY head sizes (key size != value size, sizes that are
//                      not 64 or 128), any element type including fp32, packed or paged keys, and any mix of
//                      prompt portions and single tokens in one launch. fp32 scores, softmax and accumulation.
//                      Optional: a sliding window, scores capped by cap * tanh(s / cap), a sink logit per head that
//                      joins the softmax denominator without a value, an output gate sigmoid(logit) per (token, head).
//   linear_recurrence  S_t = a_t S_(t-1) + k_t (b_t v_t)^T, o_t = S_t^T q_t (+ d v_t) per head with the state S
//                      [key size x value size] held in fp32 registers and carried between steps in a slot.
//                      Three forms: a constant decay per head (lightning attention), a decay and a step size
//                      computed per token from a projected dt (the selective state-space form of Mamba-2), or a
//                      forget gate per key channel that also decides what is written (k = 1 - f: the tied form
//                      of HGRN2), S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T.
#include "seq_common.cuh"

namespace b200 {

// ------------------------------------------------------------------ generic attention
// One CTA = 8 warps = 8 "rows" of one (sequence, kv head): row r is query token r / rep, query head
// g * rep + r % rep (rep = H / G), so that the CTA's rows share every key tile. Keys are staged 32 at a
// time in shared memory as fp32; lane j scores key j, then each lane owns value channels lane, lane+32, ...
constexpr int kAttnRows = 8;
constexpr int kAttnKeys = 32;
constexpr int kAttnMaxVChunks = 16;    // value size <= 512

template <typename T>
__global__ void __launch_bounds__(kAttnRows * 32)
attn_generic_kernel(T* __restrict__ out, const T* __restrict__ q, int64_t q_stride, const T* __restrict__ k,
                    int64_t k_stride, const T* __restrict__ v, int64_t v_stride,
                    const int* __restrict__ block_tables, int bt_stride, int block_size,
                    const int* __restrict__ cu_q, const int* __restrict__ cu_k, const int* __restrict__ ctx_lens,
                    int H, int G, int dim, int vdim, float scale, int window, float softcap,
                    const float* __restrict__ sink, const T* __restrict__ gate, int64_t gate_stride) {
  extern __shared__ float smem[];
  pdl_wait();
  const int s = blockIdx.z, g = blockIdx.y;
  const SeqSpan sp = seq_span(cu_q, cu_k, ctx_lens, s);
  const int rep = H / G;
  const int rows = sp.q_len * rep;
  const int r0 = blockIdx.x * kAttnRows;
  if (r0 >= rows) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kpad = dim + 1;
  float* sq = smem;                                   // [8][dim]
  float* sk = sq + kAttnRows * dim;                   // [32][dim + 1]
  // v == nullptr: the values are the first vdim columns of the key rows (one latent row serves as key and value)
  const bool v_in_k = v == nullptr;
  float* sv = v_in_k ? sk : sk + kAttnKeys * kpad;    // [32][vdim]
  const int vpad = v_in_k ? kpad : vdim;

  const int r = r0 + warp;
  const bool live = r < rows;
  const int tok = live ? r / rep : 0, head = g * rep + (live ? r % rep : 0);
  const int pos = sp.first_pos() + tok;               // this row sees keys lo .. pos
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (live) {
    const T* qr = q + (int64_t)(sp.q_start + tok) * q_stride + (int64_t)head * dim;
    for (int i = lane; i < dim; i += 32) sq[warp * dim + i] = to_f32<T>(qr[i]);
  }
  const int last_row = min(r0 + kAttnRows, rows) - 1;
  const int max_pos = sp.first_pos() + last_row / rep;
  const int64_t k_base = cu_k != nullptr && block_tables == nullptr ? cu_k[s] : 0;

  // a sink is one more entry of the softmax that has a logit and no value: the running state starts from it
  float m = sink != nullptr ? sink[head] : -INFINITY, l = sink != nullptr ? 1.f : 0.f, acc[kAttnMaxVChunks];
#pragma unroll
  for (int c = 0; c < kAttnMaxVChunks; ++c) acc[c] = 0.f;

  const int min_pos = sp.first_pos() + r0 / rep;
  const int first_key = window > 0 ? max(0, min_pos - window + 1) : 0;
  for (int j0 = first_key; j0 <= max_pos; j0 += kAttnKeys) {
    __syncthreads();                                  // previous tile fully consumed (and sq written)
    const int nk = min(kAttnKeys, max_pos + 1 - j0);
    for (int e = threadIdx.x; e < nk * dim; e += blockDim.x) {
      const int j = e / dim, i = e - j * dim;
      const int key = j0 + j;
      const int64_t row = block_tables != nullptr
                              ? (int64_t)block_tables[(int64_t)s * bt_stride + key / block_size] * block_size + key % block_size
                              : k_base + key;
      sk[j * kpad + i] = to_f32<T>(k[row * k_stride + (int64_t)g * dim + i]);
    }
    for (int e = threadIdx.x; e < (v_in_k ? 0 : nk * vdim); e += blockDim.x) {
      const int j = e / vdim, i = e - j * vdim;
      const int key = j0 + j;
      const int64_t row = block_tables != nullptr
                              ? (int64_t)block_tables[(int64_t)s * bt_stride + key / block_size] * block_size + key % block_size
                              : k_base + key;
      sv[j * vdim + i] = to_f32<T>(v[row * v_stride + (int64_t)g * vdim + i]);
    }
    __syncthreads();
    if (!live || j0 > pos || j0 + nk <= lo) continue;
    float sc = -INFINITY;
    if (lane < nk && j0 + lane <= pos && j0 + lane >= lo) {
      float d = 0.f;
      const float* kr = sk + lane * kpad;
      const float* qr = sq + warp * dim;
      for (int i = 0; i < dim; ++i) d += qr[i] * kr[i];
      sc = d * scale;
      if (softcap > 0.f) sc = softcap * tanhf(sc / softcap);
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float corr = expf(m - m_new);               // m = -inf on the first tile: exp(-inf) = 0
    const float p = sc == -INFINITY ? 0.f : expf(sc - m_new);
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int c = 0; c < kAttnMaxVChunks; ++c) acc[c] *= corr;
    for (int j = 0; j < nk; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
#pragma unroll
      for (int c = 0; c < kAttnMaxVChunks; ++c) {
        const int i = lane + 32 * c;
        if (i < vdim) acc[c] += pj * sv[j * vpad + i];
      }
    }
  }
  if (!live) return;
  T* o = out + (int64_t)(sp.q_start + tok) * ((int64_t)H * vdim) + (int64_t)head * vdim;
  float inv = 1.0f / l;
  if (gate != nullptr) inv *= sigmoid_f(to_f32<T>(gate[(int64_t)(sp.q_start + tok) * gate_stride + head]));
#pragma unroll
  for (int c = 0; c < kAttnMaxVChunks; ++c) {
    const int i = lane + 32 * c;
    if (i < vdim) o[i] = from_f32<T>(acc[c] * inv);
  }
}

// ------------------------------------------------------------------ linear recurrence with an fp32 state
// One CTA = 128 threads works on one (sequence, head) and a band of value columns. A thread owns ONE value column
// and KPT <= 64 key rows of the state in registers (all rows when kdim <= 64; 2 or 4 adjacent lanes share a column
// above that, one or two shuffles per token). Per token it reads k and q as float4 broadcasts from shared memory -- every lane of a warp reads the same
// address -- and its own value, and does KPT updates S <- a S + k v and KPT output terms: the loop is fp32-issue
// bound, and state rows are read and written as full 128-byte
// lines (lanes = consecutive columns). Key rows past kdim and columns past vdim are zero-padded in shared memory,
// so the inner loop has no bounds tests. Tokens are staged kRecTok at a time; the next batch is fetched into
// registers while the current one is consumed.
constexpr int kRecTok = 8;

// silu for 16-bit activations: its result is rounded to 8 or 11 bits, the fast exponential is good to ~21
__device__ __forceinline__ float silu_fast(float x) { return __fdividef(x, 1.0f + __expf(-x)); }

struct RecParams {
  const void *q, *k, *v;            // q, k: [tokens, groups * kdim] of type T; v: [tokens, H * vdim] of type TV
  int64_t q_stride, k_stride, v_stride;
  float* out;                       // [tokens, H * vdim] fp32
  float* state;                     // [slots, H, kdim, vdim] fp32 or nullptr (start from zero, keep nothing)
  const int *state_slots, *cu_q, *cu_k, *ctx_lens;
  int H, groups, kdim, vdim;
  int mode;                         // 0: constant decay per head; 1: selective (dt); 2: `k` holds a forget gate f per
                                    //    key channel (fp32): S <- diag(f) S + (1 - f) v^T
  int act_silu;                     // silu on q, k, v as they are read (mode 0)
  const float* decay;               // mode 0: [H]
  const void* dt;                   // mode 1: [tokens, H] element type T, before bias and softplus
  int64_t dt_stride;
  const float *dt_bias, *a_log, *d_skip;   // mode 1: [H] each
};

template <typename T, typename TV, int KPT, int NS>
__global__ void __launch_bounds__(128)
linear_recurrence_kernel(const RecParams P) {
  extern __shared__ __align__(16) float smem[];
  pdl_wait();
  constexpr int KS = KPT;                            // slice stride (padding it against the 2-way bank conflict of
                                                     // the NS broadcasts cost more in index arithmetic than it saved)
  constexpr int KP = NS * KS;                        // row of padded keys
  constexpr int CC = 128 / NS;                       // value columns per CTA
  const int s = blockIdx.z, h = blockIdx.y;
  const SeqSpan sp = seq_span(P.cu_q, P.cu_k, P.ctx_lens, s);
  if (sp.q_len == 0) return;
  const int kdim = P.kdim, vdim = P.vdim;
  const int ksl = threadIdx.x % NS;                  // key slice: rows ksl*KPT .. ksl*KPT + KPT - 1
  const int cl = threadIdx.x / NS;                   // column within the CTA's band
  const int c0 = blockIdx.x * CC;                    // first column of the band
  const int col = c0 + cl;
  const bool col_ok = col < vdim;
  // a warp none of whose columns exist only helps with the staging (warp-uniform, so shuffles stay legal)
  const bool warp_live = c0 + (int)((threadIdx.x & ~31u) / NS) < vdim;
  const int grp = h / (P.H / P.groups);
  float* sq = smem;                                  // [kRecTok][KP]
  float* skk = sq + kRecTok * KP;                    // [kRecTok][KP]
  float* sx = skk + kRecTok * KP;                    // [kRecTok][CC]
  float* sa = sx + kRecTok * CC;                     // [kRecTok] decay of the step
  float* sdt = sa + kRecTok;                         // [kRecTok] step size (1 for a constant decay)

  float S[KPT];
  float* slot = P.state != nullptr
                    ? P.state + (((int64_t)P.state_slots[s] * P.H + h) * kdim) * (int64_t)vdim
                    : nullptr;
  const bool carried = slot != nullptr && sp.first_pos() > 0;
#pragma unroll
  for (int r = 0; r < KPT; ++r) {
    const int i = ksl * KPT + r;
    S[r] = (carried && col_ok && i < kdim) ? slot[(int64_t)i * vdim + col] : 0.f;
  }
  const T* q = (const T*)P.q + (int64_t)grp * kdim;
  const T* k = (const T*)P.k + (int64_t)grp * kdim;
  const TV* v = (const TV*)P.v + (int64_t)h * vdim + c0;
  const T* dt = (const T*)P.dt;
  const float a_const = P.mode == 0 ? P.decay[h] : 0.f;
  const float rate = P.mode == 1 ? expf(P.a_log[h]) : 0.f;
  const float dt_b = P.mode == 1 ? P.dt_bias[h] : 0.f;
  const float d_skip = P.mode == 1 ? P.d_skip[h] : 0.f;
  const int vcols = min(CC, vdim - c0);

  constexpr int NQ = (kRecTok * KP + 127) / 128;     // q (and k) elements per thread per batch
  constexpr int NV = kRecTok * CC / 128;
  T pq[NQ], pk[NQ], pdt = from_f32<T>(0.f);
  TV pv[NV];
  auto fetch = [&](int t0) {
    const int nt = min(kRecTok, sp.q_len - t0);
    const int64_t tok0 = sp.q_start + t0;
#pragma unroll
    for (int n = 0; n < NQ; ++n) {
      const int e = threadIdx.x + n * 128;
      const int tt = e / KP, w = e % KP;
      const int i = (w / KS) * KPT + w % KS;              // key row of this shared-memory word (padding: none)
      const bool ok = tt < nt && w % KS < KPT && i < kdim;
      pq[n] = ok ? q[(tok0 + tt) * P.q_stride + i] : from_f32<T>(0.f);
      pk[n] = ok ? k[(tok0 + tt) * P.k_stride + i] : from_f32<T>(0.f);
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = threadIdx.x + n * 128;
      const int tt = e / CC, c = e % CC;
      pv[n] = (tt < nt && c < vcols) ? v[(tok0 + tt) * P.v_stride + c] : from_f32<TV>(0.f);
    }
    if (P.mode == 1 && threadIdx.x < nt) pdt = dt[(tok0 + threadIdx.x) * P.dt_stride + h];
  };
  auto stage = [&](int t0) {                         // registers -> shared memory, activations applied once
    const int nt = min(kRecTok, sp.q_len - t0);
#pragma unroll
    for (int n = 0; n < NQ; ++n) {
      const int e = threadIdx.x + n * 128;
      float qv = to_f32<T>(pq[n]), kv = to_f32<T>(pk[n]);
      // the activation's result is an activation of the model's element type (as in the 16-token form, whose
      // tensor-core operands are bf16 values); silu(0) = 0: the padding stays zero
      if (P.act_silu) {
        qv = sizeof(T) == 2 ? silu_fast(qv) : silu_f(qv);
        kv = sizeof(T) == 2 ? silu_fast(kv) : silu_f(kv);
        qv = to_f32<T>(from_f32<T>(qv)), kv = to_f32<T>(from_f32<T>(kv));
      }
      if (e < kRecTok * KP) {
        sq[e] = qv;
        skk[e] = kv;
      }
    }
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int e = threadIdx.x + n * 128;
      float x = to_f32<TV>(pv[n]);
      if (P.act_silu) x = to_f32<TV>(from_f32<TV>(sizeof(TV) == 2 ? silu_fast(x) : silu_f(x)));
      sx[e] = x;
    }
    if (threadIdx.x < nt) {
      float a = a_const, step = 1.f;
      if (P.mode == 1) {
        step = softplus_f(to_f32<T>(pdt) + dt_b);
        a = expf(-rate * step);
      }
      sa[threadIdx.x] = a;
      sdt[threadIdx.x] = step;
    }
  };

  fetch(0);
  for (int t0 = 0; t0 < sp.q_len; t0 += kRecTok) {
    const int nt = min(kRecTok, sp.q_len - t0);
    __syncthreads();                                 // the previous batch has been consumed
    stage(t0);
    __syncthreads();
    if (t0 + kRecTok < sp.q_len) fetch(t0 + kRecTok);
    if (!warp_live) continue;
    float* outp = P.out + (int64_t)(sp.q_start + t0) * ((int64_t)P.H * vdim) + (int64_t)h * vdim + col;
    for (int tt = 0; tt < nt; ++tt) {
      const float a = sa[tt], x = sx[tt * CC + cl], vj = x * sdt[tt];
      const float4* q4 = reinterpret_cast<const float4*>(sq + tt * KP + ksl * KS);
      const float4* k4 = reinterpret_cast<const float4*>(skk + tt * KP + ksl * KS);
      float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
      if (P.mode == 2) {                             // f S + (1 - f) v = v + f (S - v): the gate is the staged `k`
#pragma unroll
        for (int r4 = 0; r4 < KPT / 4; ++r4) {
          const float4 f4 = k4[r4], qq = q4[r4];
          S[r4 * 4 + 0] = fmaf(f4.x, S[r4 * 4 + 0] - vj, vj);
          o0 += S[r4 * 4 + 0] * qq.x;
          S[r4 * 4 + 1] = fmaf(f4.y, S[r4 * 4 + 1] - vj, vj);
          o1 += S[r4 * 4 + 1] * qq.y;
          S[r4 * 4 + 2] = fmaf(f4.z, S[r4 * 4 + 2] - vj, vj);
          o2 += S[r4 * 4 + 2] * qq.z;
          S[r4 * 4 + 3] = fmaf(f4.w, S[r4 * 4 + 3] - vj, vj);
          o3 += S[r4 * 4 + 3] * qq.w;
        }
      } else {
#pragma unroll
      for (int r4 = 0; r4 < KPT / 4; ++r4) {
        const float4 kq = k4[r4], qq = q4[r4];
        S[r4 * 4 + 0] = a * S[r4 * 4 + 0] + kq.x * vj;
        o0 += S[r4 * 4 + 0] * qq.x;
        S[r4 * 4 + 1] = a * S[r4 * 4 + 1] + kq.y * vj;
        o1 += S[r4 * 4 + 1] * qq.y;
        S[r4 * 4 + 2] = a * S[r4 * 4 + 2] + kq.z * vj;
        o2 += S[r4 * 4 + 2] * qq.z;
        S[r4 * 4 + 3] = a * S[r4 * 4 + 3] + kq.w * vj;
        o3 += S[r4 * 4 + 3] * qq.w;
      }
      }
      float o = (o0 + o1) + (o2 + o3);
#pragma unroll
      for (int off = 1; off < NS; off <<= 1) o += __shfl_xor_sync(0xffffffffu, o, off);
      if (ksl == 0 && col_ok) {
        if (P.mode == 1) o += d_skip * x;
        outp[(int64_t)tt * ((int64_t)P.H * vdim)] = o;
      }
    }
  }
  if (slot != nullptr && col_ok) {
#pragma unroll
    for (int r = 0; r < KPT; ++r) {
      const int i = ksl * KPT + r;
      if (i < kdim) slot[(int64_t)i * vdim + col] = S[r];
    }
  }
}

template <typename T, typename TV, int KPT, int NS>
static void recurrence_launch_as(const RecParams& P, int num_seqs, cudaStream_t stream) {
  constexpr int CC = 128 / NS;
  const dim3 grid((P.vdim + CC - 1) / CC, P.H, num_seqs);
  const size_t smem = (size_t)(2 * kRecTok * NS * KPT + kRecTok * CC + 2 * kRecTok) * sizeof(float);
  launch_pdl(linear_recurrence_kernel<T, TV, KPT, NS>, grid, dim3(128), smem, stream, P);
}

// ------------------------------------------------------------------ the same recurrence, 16 tokens at a time
// Prompt portions of bf16 models. With c_i = sum_{s<=i} log a_s inside a chunk of 16 tokens (S0 = state before it):
//   o_i = e^{c_i} S0^T q_i + sum_{j<=i} e^{c_i - c_j} b_j (q_i . k_j) v_j          S16 = e^{c_15} S0 + sum_j e^{c_15 - c_j} b_j k_j v_j^T
// -- three small matrix products per chunk on the tensor cores (mma.sync m16n8k16, fp32 accumulation). The
// 32-bit rule of the recurrence is kept: q, k, v are bf16 values already (exact operands), and every fp32 operand
// (the decayed scores, the state, the decayed values) enters the tensor core as the sum of three bf16 terms
// (hi + mid + lo, 24 bits), so each product is accurate to fp32 rounding. One CTA = one (sequence, head); warp w
// keeps rows 16w .. 16w+15 of S^T [vdim x kdim] as accumulator fragments, which are at the same time the A
// fragments of S^T q (the layout identity that flash attention uses for P V). Sizes are zero-padded to
// kdim <= D (template, 32 / 64 / 128) and vdim <= 128 in shared memory.
__device__ __forceinline__ void split3(float x, uint32_t& hi, uint32_t& mid, uint32_t& lo) {
  const __nv_bfloat16 h = __float2bfloat16_rn(x);
  const float r1 = x - __bfloat162float(h);
  const __nv_bfloat16 m = __float2bfloat16_rn(r1);
  const __nv_bfloat16 l = __float2bfloat16_rn(r1 - __bfloat162float(m));
  hi = __bfloat16_as_ushort(h), mid = __bfloat16_as_ushort(m), lo = __bfloat16_as_ushort(l);
}
// two fp32 -> three packed bf16 pairs (first value in the low half)
__device__ __forceinline__ void split3x2(float x, float y, uint32_t (&w)[3]) {
  uint32_t a[3], b[3];
  split3(x, a[0], a[1], a[2]);
  split3(y, b[0], b[1], b[2]);
#pragma unroll
  for (int i = 0; i < 3; ++i) w[i] = a[i] | (b[i] << 16);
}
__device__ __forceinline__ uint32_t bf16_bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float bits_f32(uint32_t b16) { return __uint_as_float(b16 << 16); }

constexpr int kChunk = 16;

// VEC: q, k, v rows start on 16-byte boundaries (strides, sizes and slice offsets % 8 == 0): the tiles of the next
// chunk are copied global -> shared with cp.async while the current chunk is computed (two sets of tiles).
template <int D, bool VEC>
__global__ void __launch_bounds__(256)
chunk_recurrence_kernel(const RecParams P) {
  using T = __nv_bfloat16;
  constexpr int QS = D + 8;                           // row stride (elements) of the q / k tiles: conflict-free
  constexpr int VS = 128 + 8;
  constexpr int NB = VEC ? 2 : 1;
  __shared__ __align__(16) unsigned short sQb[NB][kChunk * QS], sKb[NB][kChunk * QS], sVb[NB][kChunk * VS];
  __shared__ float sCum[kChunk], sDt[kChunk];
  __shared__ float sO[kChunk * 129];
  pdl_wait();
  const int s = blockIdx.z, h = blockIdx.y;
  const SeqSpan sp = seq_span(P.cu_q, P.cu_k, P.ctx_lens, s);
  if (sp.q_len == 0) return;
  const int kdim = P.kdim, vdim = P.vdim;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nthreads = blockDim.x;
  const int g = lane >> 2, t = lane & 3;
  const int r0 = warp * 16;                           // first row (value channel) of this warp's slab of S^T
  const int grp = h / (P.H / P.groups);
  const T* q = (const T*)P.q + (int64_t)grp * kdim;
  const T* k = (const T*)P.k + (int64_t)grp * kdim;
  const T* v = (const T*)P.v + (int64_t)h * vdim;
  const T* dt = (const T*)P.dt;
  const float log_a_const = P.mode == 0 ? fmaxf(logf(P.decay[h]), -60.f) : 0.f;   // e^-60: nothing survives a step
  const float rate = P.mode == 1 ? expf(P.a_log[h]) : 0.f;
  const float dt_b = P.mode == 1 ? P.dt_bias[h] : 0.f;
  const float d_skip = P.mode == 1 ? P.d_skip[h] : 0.f;

  // S^T slab: n-tile n = key columns 8n .. 8n+7; [0],[1]: row r0+g, cols 8n+2t, +1; [2],[3]: row r0+g+8
  float S[D / 8][4];
  float* slot = P.state != nullptr
                    ? P.state + (((int64_t)P.state_slots[s] * P.H + h) * kdim) * (int64_t)vdim
                    : nullptr;
  const bool carried = slot != nullptr && sp.first_pos() > 0;
#pragma unroll
  for (int n = 0; n < D / 8; ++n)
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int row = r0 + g + (c >> 1) * 8, col = 8 * n + 2 * t + (c & 1);
      S[n][c] = (carried && row < vdim && col < kdim) ? slot[(int64_t)col * vdim + row] : 0.f;
    }

  // asynchronous copy of the raw tiles of chunk c0 into buffer `buf` (zero-filled past the chunk / the sizes)
  auto copy_async = [&](int c0, int buf) {
    const int nt = min(kChunk, sp.q_len - c0);
    const int64_t tok0 = sp.q_start + c0;
    for (int e = threadIdx.x; e < kChunk * (D / 8); e += nthreads) {
      const int j = e / (D / 8), i = (e % (D / 8)) * 8;
      const bool ok = j < nt && i < kdim;
      const int64_t tok = ok ? tok0 + j : sp.q_start;
      cp_async_16(smem_u32(&sQb[buf][j * QS + i]), q + tok * P.q_stride + (ok ? i : 0), ok);
      cp_async_16(smem_u32(&sKb[buf][j * QS + i]), k + tok * P.k_stride + (ok ? i : 0), ok);
    }
    for (int e = threadIdx.x; e < kChunk * 16; e += nthreads) {
      const int j = e >> 4, i = (e & 15) * 8;
      const bool ok = j < nt && i < vdim;
      const int64_t tok = ok ? tok0 + j : sp.q_start;
      cp_async_16(smem_u32(&sVb[buf][j * VS + i]), v + tok * P.v_stride + (ok ? i : 0), ok);
    }
    cp_async_commit();
  };
  float dt_next = 0.f;                                // this thread's token of the next chunk (threads < 16)
  auto fetch_dt = [&](int c0) {
    dt_next = 0.f;
    if (P.mode == 1 && threadIdx.x < kChunk && c0 + (int)threadIdx.x < sp.q_len)
      dt_next = __bfloat162float(dt[(sp.q_start + c0 + threadIdx.x) * P.dt_stride + h]);
  };
  if (VEC) copy_async(0, 0);
  fetch_dt(0);

  for (int c0 = 0, it = 0; c0 < sp.q_len; c0 += kChunk, ++it) {
    const int nt = min(kChunk, sp.q_len - c0);
    const int64_t tok0 = sp.q_start + c0;
    const int buf = VEC ? (it & 1) : 0;
    unsigned short* sQ = sQb[buf];
    unsigned short* sK = sKb[buf];
    unsigned short* sV = sVb[buf];
    if (VEC) cp_async_wait<0>();
    __syncthreads();                                  // this chunk's tiles have landed; the previous chunk is consumed
    if (VEC) {
      if (c0 + kChunk < sp.q_len) copy_async(c0 + kChunk, buf ^ 1);
      if (P.act_silu) {                               // activation in place, 8 values per step
        for (int e = threadIdx.x; e < kChunk * (D / 8) * 2 + kChunk * 16; e += nthreads) {
          unsigned short* p;
          if (e < kChunk * (D / 8)) p = sQ + (e / (D / 8)) * QS + (e % (D / 8)) * 8;
          else if (e < 2 * kChunk * (D / 8)) p = sK + ((e - kChunk * (D / 8)) / (D / 8)) * QS + ((e - kChunk * (D / 8)) % (D / 8)) * 8;
          else p = sV + ((e - 2 * kChunk * (D / 8)) >> 4) * VS + ((e - 2 * kChunk * (D / 8)) & 15) * 8;
          float f[8];
          load8<T>(reinterpret_cast<const T*>(p), f);
#pragma unroll
          for (int u = 0; u < 8; ++u) f[u] = silu_fast(f[u]);
          store8<T>(reinterpret_cast<T*>(p), f);
        }
      }
    } else {
      for (int e = threadIdx.x; e < kChunk * D; e += nthreads) {
        const int j = e / D, i = e % D;
        float qv = 0.f, kv = 0.f;
        if (j < nt && i < kdim) {
          qv = __bfloat162float(q[(tok0 + j) * P.q_stride + i]);
          kv = __bfloat162float(k[(tok0 + j) * P.k_stride + i]);
          if (P.act_silu) qv = silu_fast(qv), kv = silu_fast(kv);
        }
        sQ[j * QS + i] = (unsigned short)bf16_bits(qv);
        sK[j * QS + i] = (unsigned short)bf16_bits(kv);
      }
      for (int e = threadIdx.x; e < kChunk * 128; e += nthreads) {
        const int j = e >> 7, i = e & 127;
        float x = 0.f;
        if (j < nt && i < vdim) {
          x = __bfloat162float(v[(tok0 + j) * P.v_stride + i]);
          if (P.act_silu) x = silu_fast(x);
        }
        sV[j * VS + i] = (unsigned short)bf16_bits(x);
      }
    }
    if (warp == 0) {                                  // log-decay of every token and its prefix sum; step sizes
      float la = 0.f, step = 1.f;                     // a padded token neither decays nor adds
      if (lane < nt) {
        la = log_a_const;
        if (P.mode == 1) {
          step = softplus_f(dt_next + dt_b);
          la = -rate * step;
        }
      }
#pragma unroll
      for (int off = 1; off < kChunk; off <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, la, off);
        if (lane >= off) la += up;
      }
      if (lane < kChunk) {
        sCum[lane] = la;
        sDt[lane] = step;
      }
    }
    fetch_dt(c0 + kChunk);
    __syncthreads();
    if (r0 < vdim) {                                  // (every warp of the CTA, by the launch's block size)
      // ---- 1. scores q_i . k_j : rows i = g, g+8; columns j = 8*nj + 2t, +1
      float qk[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const int kk = 16 * ks + 2 * t;
        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(sQ + g * QS + kk);
        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(sQ + (g + 8) * QS + kk);
        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(sQ + g * QS + kk + 8);
        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(sQ + (g + 8) * QS + kk + 8);
#pragma unroll
        for (int nj = 0; nj < 2; ++nj) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(sK + (8 * nj + g) * QS + kk);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(sK + (8 * nj + g) * QS + kk + 8);
          mma_16816<T>(qk[nj], a0, a1, a2, a3, b0, b1);
        }
      }
      // ---- 2. decayed, causal: p_ij = (j <= i) e^{c_i - c_j} b_j (q_i . k_j)
      const float ci[2] = {sCum[g], sCum[g + 8]};
#pragma unroll
      for (int nj = 0; nj < 2; ++nj)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int i = g + (c >> 1) * 8, j = 8 * nj + 2 * t + (c & 1);
          qk[nj][c] = j <= i ? qk[nj][c] * expf(ci[c >> 1] - sCum[j]) * sDt[j] : 0.f;
        }
      // ---- 3. o^T (rows: value channels, columns: tokens i) = V^T P^T
      uint32_t va[4];                                 // V^T fragment: rows r0+g / +8, k = tokens 2t,2t+1 / 2t+8,2t+9
      {
        const unsigned short* vp = sV + r0 + g;
        va[0] = vp[(2 * t) * VS] | ((uint32_t)vp[(2 * t + 1) * VS] << 16);
        va[1] = vp[(2 * t) * VS + 8] | ((uint32_t)vp[(2 * t + 1) * VS + 8] << 16);
        va[2] = vp[(2 * t + 8) * VS] | ((uint32_t)vp[(2 * t + 9) * VS] << 16);
        va[3] = vp[(2 * t + 8) * VS + 8] | ((uint32_t)vp[(2 * t + 9) * VS + 8] << 16);
      }
      float o[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ni = 0; ni < 2; ++ni) {                // token columns i = 8*ni + g  (B[k = j][n = i] = p_ij)
        uint32_t b0[3], b1[3];
        split3x2(qk[0][2 * ni], qk[0][2 * ni + 1], b0);          // j = 2t, 2t+1
        split3x2(qk[1][2 * ni], qk[1][2 * ni + 1], b1);          // j = 2t+8, 2t+9
#pragma unroll
        for (int p = 0; p < 3; ++p) mma_16816<T>(o[ni], va[0], va[1], va[2], va[3], b0[p], b1[p]);
      }
      // ---- 4. carried part: o^T += (S^T Q^T) scaled per token column by e^{c_i}
      float oi[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a0[3], a1[3], a2[3], a3[3];
        split3x2(S[2 * ks][0], S[2 * ks][1], a0);
        split3x2(S[2 * ks][2], S[2 * ks][3], a1);
        split3x2(S[2 * ks + 1][0], S[2 * ks + 1][1], a2);
        split3x2(S[2 * ks + 1][2], S[2 * ks + 1][3], a3);
        const int kk = 16 * ks + 2 * t;
#pragma unroll
        for (int ni = 0; ni < 2; ++ni) {
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(sQ + (8 * ni + g) * QS + kk);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(sQ + (8 * ni + g) * QS + kk + 8);
#pragma unroll
          for (int p = 0; p < 3; ++p) mma_16816<T>(oi[ni], a0[p], a1[p], a2[p], a3[p], b0, b1);
        }
      }
#pragma unroll
      for (int ni = 0; ni < 2; ++ni)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int i = 8 * ni + 2 * t + (c & 1), row = r0 + g + (c >> 1) * 8;
          float val = o[ni][c] + oi[ni][c] * expf(sCum[i]);
          if (P.mode == 1) val += d_skip * bits_f32(sV[i * VS + row]);
          sO[i * 129 + row] = val;
        }
      // ---- 5. S^T <- e^{c_15} S^T + V'^T K,  v'_j = e^{c_15 - c_j} b_j v_j
      const float c_end = sCum[kChunk - 1];
      const float grow = expf(c_end);
#pragma unroll
      for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) S[n][c] *= grow;
      uint32_t wa[4][3];
      {
        const int js[4] = {2 * t, 2 * t + 1, 2 * t + 8, 2 * t + 9};
        float f[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) f[u] = expf(c_end - sCum[js[u]]) * sDt[js[u]];
        split3x2(bits_f32(va[0] & 0xffffu) * f[0], bits_f32(va[0] >> 16) * f[1], wa[0]);
        split3x2(bits_f32(va[1] & 0xffffu) * f[0], bits_f32(va[1] >> 16) * f[1], wa[1]);
        split3x2(bits_f32(va[2] & 0xffffu) * f[2], bits_f32(va[2] >> 16) * f[3], wa[2]);
        split3x2(bits_f32(va[3] & 0xffffu) * f[2], bits_f32(va[3] >> 16) * f[3], wa[3]);
      }
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {               // B[k = token j][n = key column 8n + g] = k_j
        const unsigned short* kp = sK + 8 * n + g;
        const uint32_t b0 = kp[(2 * t) * QS] | ((uint32_t)kp[(2 * t + 1) * QS] << 16);
        const uint32_t b1 = kp[(2 * t + 8) * QS] | ((uint32_t)kp[(2 * t + 9) * QS] << 16);
#pragma unroll
        for (int p = 0; p < 3; ++p) mma_16816<T>(S[n], wa[0][p], wa[1][p], wa[2][p], wa[3][p], b0, b1);
      }
    }
    __syncthreads();
    float* outp = P.out + tok0 * ((int64_t)P.H * vdim) + (int64_t)h * vdim;
    for (int e = threadIdx.x; e < nt * vdim; e += nthreads) {
      const int i = e / vdim, c = e - i * vdim;
      outp[(int64_t)i * ((int64_t)P.H * vdim) + c] = sO[i * 129 + c];
    }
  }
  if (slot != nullptr && r0 < vdim) {
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int row = r0 + g + (c >> 1) * 8, col = 8 * n + 2 * t + (c & 1);
        if (row < vdim && col < kdim) slot[(int64_t)col * vdim + row] = S[n][c];
      }
  }
}

static bool chunk_recurrence_ok(const RecParams& P, int dtype, int max_q) {
  static const bool off = [] {
    const char* e = getenv("B200_CHUNK_RECURRENCE");
    return e != nullptr && e[0] == '0';
  }();
  return !off && P.mode != 2 && dtype == B200_DTYPE_BF16 && P.cu_q != nullptr && max_q >= kChunk && P.kdim <= 128 && P.vdim <= 128;
}

static int chunk_recurrence_launch(const RecParams& P, int num_seqs, cudaStream_t stream) {
  const dim3 grid(1, P.H, num_seqs);
  const dim3 block(32 * ((P.vdim + 15) / 16));
  const bool vec = P.kdim % 8 == 0 && P.vdim % 8 == 0 && P.q_stride % 8 == 0 && P.k_stride % 8 == 0 &&
                   P.v_stride % 8 == 0 && aligned16(P.q) && aligned16(P.k) && aligned16(P.v);
#define B200_CHUNK_REC(DV)                                                                       \
  do {                                                                                           \
    if (vec) launch_pdl(chunk_recurrence_kernel<DV, true>, grid, block, 0, stream, P);           \
    else launch_pdl(chunk_recurrence_kernel<DV, false>, grid, block, 0, stream, P);              \
  } while (0)
  if (P.kdim <= 32) B200_CHUNK_REC(32);
  else if (P.kdim <= 64) B200_CHUNK_REC(64);
  else B200_CHUNK_REC(128);
#undef B200_CHUNK_REC
  return finish_launch();
}

template <typename T, typename TV = T>
static int recurrence_launch(const RecParams& P, int num_seqs, cudaStream_t stream) {
  if (P.kdim <= 16) recurrence_launch_as<T, TV, 16, 1>(P, num_seqs, stream);
  else if (P.kdim <= 32) recurrence_launch_as<T, TV, 32, 1>(P, num_seqs, stream);
  else if (P.kdim <= 64) recurrence_launch_as<T, TV, 64, 1>(P, num_seqs, stream);
  else if (P.kdim <= 128) recurrence_launch_as<T, TV, 64, 2>(P, num_seqs, stream);
  else recurrence_launch_as<T, TV, 64, 4>(P, num_seqs, stream);
  return finish_launch();
}

}  // namespace b200

using namespace b200;

extern "C" int b200_attn_generic(void* out, const void* q, int64_t q_stride, const void* k, int64_t k_stride,
                                 const void* v, int64_t v_stride, const int32_t* block_tables,
                                 int32_t bt_stride, int32_t block_size, const int32_t* cu_q,
                                 const int32_t* cu_k, const int32_t* ctx_lens, int32_t num_seqs, int32_t max_q,
                                 int32_t num_heads, int32_t num_kv_heads, int32_t dim, int32_t vdim,
                                 float scale, int32_t window, float softcap, const float* sink, const void* gate,
                                 int64_t gate_stride, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_seqs < 0 || max_q < 0 || num_heads <= 0 || num_kv_heads <= 0 || dim <= 0 || vdim <= 0 ||
                     num_heads % num_kv_heads != 0, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(vdim > 32 * kAttnMaxVChunks, B200_ERR_UNSUPPORTED);
  if (num_seqs == 0 || max_q == 0) return B200_OK;
  B200_RETURN_IF(!out || !q || !k || (cu_q == nullptr) == (ctx_lens == nullptr) || (cu_q && !cu_k),
                 B200_ERR_NULL_POINTER);
  B200_RETURN_IF(block_tables && block_size <= 0, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(window < 0 || (!v && vdim > dim), B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(!block_tables && !cu_q, B200_ERR_NULL_POINTER);       // decode rows read the paged cache
  const int rep = num_heads / num_kv_heads;
  const dim3 grid((max_q * rep + kAttnRows - 1) / kAttnRows, num_kv_heads, num_seqs);
  const size_t smem = (size_t)(kAttnRows * dim + kAttnKeys * (dim + 1) + (v ? kAttnKeys * vdim : 0)) * sizeof(float);
  B200_RETURN_IF(smem > 200 * 1024, B200_ERR_UNSUPPORTED);
  B200_DISPATCH_3(dtype, T, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(attn_generic_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_pdl(attn_generic_kernel<T>, grid, dim3(kAttnRows * 32), smem, (cudaStream_t)stream, (T*)out,
               (const T*)q, q_stride, (const T*)k, k_stride, (const T*)v, v_stride, block_tables, bt_stride,
               block_size, cu_q, cu_k, ctx_lens, num_heads, num_kv_heads, dim, vdim, scale, window, softcap, sink,
               (const T*)gate, gate_stride);
  });
  return finish_launch();
}

extern "C" int b200_linear_recurrence(float* out, const void* q, int64_t q_stride, const void* k,
                                      int64_t k_stride, const void* v, int64_t v_stride, float* state,
                                      const int32_t* state_slots, const int32_t* cu_q, const int32_t* cu_k,
                                      const int32_t* ctx_lens, int32_t num_seqs, int32_t max_q,
                                      int32_t num_heads, int32_t groups, int32_t kdim, int32_t vdim, int32_t mode,
                                      int32_t act_silu, const float* decay, const void* dt, int64_t dt_stride,
                                      const float* dt_bias, const float* a_log, const float* d_skip,
                                      int32_t qk_f32, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_seqs < 0 || num_heads <= 0 || groups <= 0 || num_heads % groups != 0 || kdim <= 0 ||
                     vdim <= 0 || mode < 0 || mode > 2, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(kdim > 256, B200_ERR_UNSUPPORTED);
  if (num_seqs == 0) return B200_OK;
  B200_RETURN_IF(!out || !q || !k || !v || (cu_q == nullptr) == (ctx_lens == nullptr) || (cu_q && !cu_k) ||
                     (state && !state_slots), B200_ERR_NULL_POINTER);
  B200_RETURN_IF(mode == 0 ? !decay : (mode == 1 && (!dt || !dt_bias || !a_log || !d_skip)), B200_ERR_NULL_POINTER);
  B200_RETURN_IF(mode == 2 && !qk_f32 && dtype != B200_DTYPE_F32, B200_ERR_BAD_DTYPE);   // the gate is fp32
  RecParams P;
  P.q = q, P.k = k, P.v = v, P.q_stride = q_stride, P.k_stride = k_stride, P.v_stride = v_stride;
  P.out = out, P.state = state, P.state_slots = state_slots, P.cu_q = cu_q, P.cu_k = cu_k, P.ctx_lens = ctx_lens;
  P.H = num_heads, P.groups = groups, P.kdim = kdim, P.vdim = vdim, P.mode = mode, P.act_silu = act_silu;
  P.decay = decay, P.dt = dt, P.dt_stride = dt_stride, P.dt_bias = dt_bias, P.a_log = a_log, P.d_skip = d_skip;
  if (qk_f32 && dtype != B200_DTYPE_F32) {           // q, k already fp32 (rotated or normalised upstream), v as projected
    B200_RETURN_IF(mode == 1, B200_ERR_UNSUPPORTED);
    if (dtype == B200_DTYPE_BF16) return recurrence_launch<float, __nv_bfloat16>(P, num_seqs, (cudaStream_t)stream);
    if (dtype == B200_DTYPE_F16) return recurrence_launch<float, __half>(P, num_seqs, (cudaStream_t)stream);
    return B200_ERR_BAD_DTYPE;
  }
  if (chunk_recurrence_ok(P, dtype, max_q)) return chunk_recurrence_launch(P, num_seqs, (cudaStream_t)stream);
  B200_DISPATCH_3(dtype, T, return recurrence_launch<T>(P, num_seqs, (cudaStream_t)stream));
  return B200_OK;
}
