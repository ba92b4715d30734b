// mixed_attn.cu -- causal softmax attention whose heads talk to each other BEFORE the softmax:
//
//   s_h(i, j) = scale (q_h,i . k_g(h),j) - slope_h (i - j)            a linear distance bias per head (optional)
//   s'_h(i, j) = sum_g talk[h][g] s_g(i, j)                            every head's score is a mix of all heads' scores
//   p_h(i, .) = exp(s'_h(i, .)) / (sum_j exp(s'_h(i, j)) + exp(sink_h))   over the visible keys; the sink has no key,
//   o_h,i = sum_j p_h(i, j) v_g(h),j                                    no value, no bias, and counts once (optional)
//
// with a sliding window (0 <= i - j < window, 0 = none), any head sizes (key size != value size allowed), any
// element type including fp32, packed or paged keys, and any mix of prompt portions and single tokens in one launch.
// Scores, mixing, softmax and accumulation are fp32.
//
// The mix needs the scores of ALL heads at a (query, key) pair, so one CTA owns TQ query tokens with all their heads:
// 8 warps share tq * H rows (row = token * H + head, RPW rows per warp, their softmax state and output accumulators in
// registers). Keys and values of ALL kv heads are staged `kt` keys at a time in shared memory as fp32. Per tile: every
// warp scores its rows (lane j = key j) into shared memory; after a barrier it mixes them (H terms per row), applies
// the mask, and does the online-softmax update and the P V product (each lane owns value channels lane, lane + 32, ...).
#include "seq_common.cuh"

namespace b200 {

constexpr int kMixWarps = 8;

struct MixAttnParams {
  void* out;                        // [tokens, H * vdim]
  const void *q, *k, *v;            // q [tokens, H, dim]; packed k [keys, G, dim], v [keys, G, vdim], or the paged caches
  int64_t q_stride, k_stride, v_stride;
  const int* block_tables;
  int bt_stride, block_size;
  const int *cu_q, *cu_k, *ctx_lens;
  int H, G, dim, vdim, window;
  float scale;
  const float* slopes;              // [H] or nullptr
  const float* talk;                // [H, H] (to, from) or nullptr: no mixing
  const float* sink;                // [H] or nullptr
  int tq, kt;                       // query tokens per CTA; keys per tile (<= 32)
};

template <typename T, int RPW, int VC>
__global__ void __launch_bounds__(kMixWarps * 32)
mixed_attn_kernel(const MixAttnParams P) {
  extern __shared__ float smem[];
  pdl_wait();
  const int s = blockIdx.y;
  const SeqSpan sp = seq_span(P.cu_q, P.cu_k, P.ctx_lens, s);
  const int t0 = blockIdx.x * P.tq;
  if (t0 >= sp.q_len) return;
  const int H = P.H, G = P.G, dim = P.dim, vdim = P.vdim, rep = H / G, kt = P.kt;
  const int ntok = min(P.tq, sp.q_len - t0);
  const int nrows = ntok * H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kpad = dim + 1;
  float* sq = smem;                                   // [tq * H][dim]
  float* sk = sq + (size_t)P.tq * H * dim;            // [kt][G][dim + 1]
  float* sv = sk + (size_t)kt * G * kpad;             // [kt][G][vdim]
  float* ss = sv + (size_t)kt * G * vdim;             // [tq * H][32] biased scores of the tile
  float* stalk = ss + (size_t)P.tq * H * 32;          // [H][H]
  float* sslope = stalk + H * H;                      // [H]

  const T* q = (const T*)P.q;
  const T* k = (const T*)P.k;
  const T* v = (const T*)P.v;
  for (int e = threadIdx.x; e < nrows * dim; e += blockDim.x) {
    const int row = e / dim, i = e - row * dim;
    const int tok = row / H, head = row - tok * H;
    sq[e] = to_f32<T>(q[(int64_t)(sp.q_start + t0 + tok) * P.q_stride + (int64_t)head * dim + i]);
  }
  for (int e = threadIdx.x; e < H * H; e += blockDim.x)
    stalk[e] = P.talk != nullptr ? P.talk[e] : (e / H == e % H ? 1.f : 0.f);
  for (int e = threadIdx.x; e < H; e += blockDim.x) sslope[e] = P.slopes != nullptr ? P.slopes[e] : 0.f;

  const int first_pos = sp.first_pos() + t0;          // position of the CTA's first token
  const int max_pos = first_pos + ntok - 1;
  const int first_key = P.window > 0 ? max(0, first_pos - P.window + 1) : 0;
  const int64_t k_base = P.cu_k != nullptr && P.block_tables == nullptr ? P.cu_k[s] : 0;

  float m[RPW], l[RPW], acc[RPW][VC];
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    m[r] = -INFINITY, l[r] = 0.f;
#pragma unroll
    for (int c = 0; c < VC; ++c) acc[r][c] = 0.f;
  }

  for (int j0 = first_key; j0 <= max_pos; j0 += kt) {
    __syncthreads();                                  // the previous tile is consumed (and sq, stalk are written)
    const int nk = min(kt, max_pos + 1 - j0);
    for (int e = threadIdx.x; e < nk * G * dim; e += blockDim.x) {
      const int j = e / (G * dim), c = e - j * (G * dim);
      const int key = j0 + j;
      const int64_t row = P.block_tables != nullptr
                              ? (int64_t)P.block_tables[(int64_t)s * P.bt_stride + key / P.block_size] * P.block_size +
                                    key % P.block_size
                              : k_base + key;
      sk[(size_t)(j * G + c / dim) * kpad + c % dim] = to_f32<T>(k[row * P.k_stride + c]);
    }
    for (int e = threadIdx.x; e < nk * G * vdim; e += blockDim.x) {
      const int j = e / (G * vdim), c = e - j * (G * vdim);
      const int key = j0 + j;
      const int64_t row = P.block_tables != nullptr
                              ? (int64_t)P.block_tables[(int64_t)s * P.bt_stride + key / P.block_size] * P.block_size +
                                    key % P.block_size
                              : k_base + key;
      sv[(size_t)j * G * vdim + c] = to_f32<T>(v[row * P.v_stride + c]);
    }
    __syncthreads();
    // ---- 1. scale q.k minus the distance bias, every row of the CTA, lane = key
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int row = warp + kMixWarps * r;
      if (row >= nrows) continue;
      const int tok = row / H, head = row - tok * H, g = head / rep;
      float sc = 0.f;
      if (lane < nk) {
        const float* kr = sk + (size_t)(lane * G + g) * kpad;
        const float* qr = sq + (size_t)row * dim;
        float d = 0.f;
        for (int i = 0; i < dim; ++i) d += qr[i] * kr[i];
        sc = d * P.scale - sslope[head] * (float)(first_pos + tok - (j0 + lane));
      }
      ss[row * 32 + lane] = sc;
    }
    __syncthreads();
    // ---- 2. mix the heads, mask, online softmax, P V
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int row = warp + kMixWarps * r;
      if (row >= nrows) continue;
      const int tok = row / H, head = row - tok * H, g = head / rep;
      const int pos = first_pos + tok;
      const int lo = P.window > 0 ? max(0, pos - P.window + 1) : 0;
      const int key = j0 + lane;
      float sc = -INFINITY;
      if (lane < nk && key <= pos && key >= lo) {
        const float* tr = stalk + head * H;
        const float* sr = ss + (size_t)tok * H * 32 + lane;
        float d = 0.f;
        for (int g2 = 0; g2 < H; ++g2) d += tr[g2] * sr[g2 * 32];
        sc = d;
      }
      const float tile_max = warp_max(sc);
      if (tile_max == -INFINITY) continue;            // no key of this tile is visible to the row (warp-uniform)
      const float m_new = fmaxf(m[r], tile_max);
      const float corr = expf(m[r] - m_new);          // m = -inf before the first visible key: exp(-inf) = 0
      const float p = sc == -INFINITY ? 0.f : expf(sc - m_new);
      l[r] = l[r] * corr + warp_sum(p);
      m[r] = m_new;
#pragma unroll
      for (int c = 0; c < VC; ++c) acc[r][c] *= corr;
      const float* vb = sv + (size_t)g * vdim;
      for (int j = 0; j < nk; ++j) {
        const float pj = __shfl_sync(0xffffffffu, p, j);
        const float* vr = vb + (size_t)j * G * vdim;
#pragma unroll
        for (int c = 0; c < VC; ++c) {
          const int i = lane + 32 * c;
          if (i < vdim) acc[r][c] += pj * vr[i];
        }
      }
    }
  }
  T* out = (T*)P.out;
#pragma unroll
  for (int r = 0; r < RPW; ++r) {
    const int row = warp + kMixWarps * r;
    if (row >= nrows) continue;
    const int tok = row / H, head = row - tok * H;
    float lr = l[r], mul = 1.f;
    if (P.sink != nullptr) {                          // one more term in the denominator, no value
      const float sk_h = P.sink[head];
      const float m2 = fmaxf(m[r], sk_h);
      mul = expf(m[r] - m2);
      lr = lr * mul + expf(sk_h - m2);
    }
    const float inv = mul / lr;
    T* o = out + (int64_t)(sp.q_start + t0 + tok) * ((int64_t)H * vdim) + (int64_t)head * vdim;
#pragma unroll
    for (int c = 0; c < VC; ++c) {
      const int i = lane + 32 * c;
      if (i < vdim) o[i] = from_f32<T>(acc[r][c] * inv);
    }
  }
}

template <typename T, int RPW, int VC>
static void mixed_attn_launch(const MixAttnParams& P, dim3 grid, size_t smem, cudaStream_t stream) {
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(mixed_attn_kernel<T, RPW, VC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  launch_pdl(mixed_attn_kernel<T, RPW, VC>, grid, dim3(kMixWarps * 32), smem, stream, P);
}

template <typename T>
static int mixed_attn_dispatch(const MixAttnParams& P, int rpw, int vc, dim3 grid, size_t smem, cudaStream_t stream) {
#define B200_MIX_CASE(R, V)                                   \
  if (rpw == R && vc == V) {                                  \
    mixed_attn_launch<T, R, V>(P, grid, smem, stream);        \
    return finish_launch();                                   \
  }
  B200_MIX_CASE(1, 2) B200_MIX_CASE(2, 2) B200_MIX_CASE(4, 2) B200_MIX_CASE(8, 2)
  B200_MIX_CASE(1, 4) B200_MIX_CASE(2, 4) B200_MIX_CASE(4, 4) B200_MIX_CASE(8, 4)
  B200_MIX_CASE(1, 8) B200_MIX_CASE(2, 8) B200_MIX_CASE(4, 8)
#undef B200_MIX_CASE
  return B200_ERR_UNSUPPORTED;
}

}  // namespace b200

using namespace b200;

extern "C" int b200_mixed_attn(void* out, const void* q, int64_t q_stride, const void* k, int64_t k_stride,
                               const void* v, int64_t v_stride, const int32_t* block_tables, int32_t bt_stride,
                               int32_t block_size, const int32_t* cu_q, const int32_t* cu_k,
                               const int32_t* ctx_lens, int32_t num_seqs, int32_t max_q, int32_t num_heads,
                               int32_t num_kv_heads, int32_t dim, int32_t vdim, float scale, int32_t window,
                               const float* slopes, const float* talk, const float* sink, int32_t dtype,
                               b200_stream_t stream) {
  B200_RETURN_IF(num_seqs < 0 || max_q < 0 || num_heads <= 0 || num_kv_heads <= 0 || dim <= 0 || vdim <= 0 ||
                     num_heads % num_kv_heads != 0 || window < 0, B200_ERR_BAD_SHAPE);
  if (num_seqs == 0 || max_q == 0) return B200_OK;
  B200_RETURN_IF(!out || !q || !k || !v || (cu_q == nullptr) == (ctx_lens == nullptr) || (cu_q && !cu_k),
                 B200_ERR_NULL_POINTER);
  B200_RETURN_IF(block_tables && block_size <= 0, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(!block_tables && !cu_q, B200_ERR_NULL_POINTER);       // single-token rows read the paged cache
  const int vc = vdim <= 64 ? 2 : vdim <= 128 ? 4 : 8;
  B200_RETURN_IF(vdim > 256, B200_ERR_UNSUPPORTED);
  const int max_rpw = vc == 8 ? 4 : 8;                 // rows per warp x value chunks per lane <= 32 accumulators
  B200_RETURN_IF(num_heads > kMixWarps * max_rpw, B200_ERR_UNSUPPORTED);
  int tq = (kMixWarps * max_rpw) / num_heads;          // as many tokens per CTA as the registers allow, at most 8
  if (tq > 8) tq = 8;
  if (tq > max_q) tq = max_q;
  int rpw = 1;
  while (rpw * kMixWarps < tq * num_heads) rpw <<= 1;
  MixAttnParams P;
  P.out = out, P.q = q, P.k = k, P.v = v, P.q_stride = q_stride, P.k_stride = k_stride, P.v_stride = v_stride;
  P.block_tables = block_tables, P.bt_stride = bt_stride, P.block_size = block_size;
  P.cu_q = cu_q, P.cu_k = cu_k, P.ctx_lens = ctx_lens;
  P.H = num_heads, P.G = num_kv_heads, P.dim = dim, P.vdim = vdim, P.window = window, P.scale = scale;
  P.slopes = slopes, P.talk = talk, P.sink = sink, P.tq = tq;
  const size_t fixed = ((size_t)tq * num_heads * (dim + 32) + (size_t)num_heads * (num_heads + 1)) * sizeof(float);
  const size_t per_key = (size_t)num_kv_heads * (dim + 1 + vdim) * sizeof(float);
  int kt = 32;
  while (kt > 1 && fixed + kt * per_key > 160 * 1024) kt >>= 1;
  B200_RETURN_IF(fixed + kt * per_key > 200 * 1024, B200_ERR_UNSUPPORTED);
  P.kt = kt;
  const size_t smem = fixed + kt * per_key;
  const dim3 grid((max_q + tq - 1) / tq, num_seqs);
  B200_DISPATCH_3(dtype, T, return mixed_attn_dispatch<T>(P, rpw, vc, grid, smem, (cudaStream_t)stream));
  return B200_OK;
}
