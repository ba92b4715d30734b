// moe_generic.cu -- the parts of a sparse mixture-of-experts layer that the tensor-core kernels of moe.cu do not
// cover: a sigmoid router with a selection bias and group-limited choice, and expert GEMMs for ANY sizes and
// element types (fp32 included), with fp32 routing weights applied in an fp32 combine.
//
//   moe_route_grouped    s = sigmoid(z); choice = s + bias; experts form `groups` equal groups of neighbours, a
//                        group scores the sum of its two largest choices, only the `keep` best groups stay in
//                        play (the others count as -inf); the top-k choices are taken and weighted by
//                        s / (sum s + 1e-20) * scale. Ties go to the lower index. fp32 throughout.
//   moe_route_grouped_softmax  s = softmax(z) over all experts; a group scores its largest s; the `keep` best groups
//                        stay in play; the top-k s are taken and weighted by s / (sum s + 1e-20) * scale.
//   moe_route_topk       the k largest of z + bias; weights = softmax over the chosen logits only. fp32 throughout.
//   moe_gemm_generic     H[pos] = silu(X[token(pos)] Wg[e]^T) * (X[token(pos)] Wu[e]^T)   (gate_up; or the clamped unit
//                        g sigmoid(alpha g) (u + 1), g = min(gate, limit), u = clamp(up, +-limit))
//                        H[pos] = act(X[token(pos)] Wu[e]^T)                               (up alone, no gate)
//                        Y[pos] = H[pos] W2[e]^T, fp32                                     (down)
//                        over the dispatch plan of moe_align (pairs sorted by expert); 32 x 64 tiles, fp32 FMA.
//   moe_combine_weighted out[t] = sum_j w[t][j] Y[pos(t, j)], accumulated in fp32, one rounding.
#include "seq_common.cuh"

namespace b200 {

constexpr int kRouteMaxExperts = 512;
constexpr int kRouteMaxTopK = 16;
constexpr int kRouteMaxGroups = 64;

// one warp per token; the token's choice scores live in shared memory
__global__ void __launch_bounds__(128)
moe_route_grouped_kernel(int32_t* __restrict__ ids, float* __restrict__ weights, const float* __restrict__ logits,
                         int64_t logit_stride, const float* __restrict__ bias, int tokens, int E, int top_k,
                         int groups, int keep, float scale, int kind) {
  extern __shared__ float smem[];                    // per warp: choice [E], s [E]
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t = (int64_t)blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  float* choice = smem + (size_t)warp * 2 * E;
  float* sg = choice + E;
  float zmax_all = -INFINITY, zsum_all = 0.f;
  if (kind == 2) {                                   // softmax over ALL experts: the row's max and sum first
    for (int e = lane; e < E; e += 32) zmax_all = fmaxf(zmax_all, logits[t * logit_stride + e]);
    zmax_all = warp_max(zmax_all);
    for (int e = lane; e < E; e += 32) zsum_all += expf(logits[t * logit_stride + e] - zmax_all);
    zsum_all = warp_sum(zsum_all);
  }
  for (int e = lane; e < E; e += 32) {
    if (kind == 2) {
      const float s = expf(logits[t * logit_stride + e] - zmax_all) / zsum_all;
      sg[e] = s;
      choice[e] = s;
    } else if (kind == 1) {                                 // the bias is part of the logit; weights: softmax over the chosen
      const float z = logits[t * logit_stride + e] + (bias != nullptr ? bias[e] : 0.f);
      sg[e] = z;
      choice[e] = z;
    } else {
      const float s = sigmoid_f(logits[t * logit_stride + e]);
      sg[e] = s;
      choice[e] = s + (bias != nullptr ? bias[e] : 0.f);
    }
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    // lane g (looping) scores group g; then `keep` rounds of arg-max over the group scores
    float gs[(kRouteMaxGroups + 31) / 32];
#pragma unroll
    for (int i = 0; i < (kRouteMaxGroups + 31) / 32; ++i) {
      const int g = lane + 32 * i;
      float a = -INFINITY, b = -INFINITY;
      if (g < groups)
        for (int e = g * per; e < (g + 1) * per; ++e) {
          const float c = choice[e];
          if (c > a) b = a, a = c;
          else if (c > b) b = c;
        }
      gs[i] = g < groups ? (per > 1 && kind != 2 ? a + b : a) : -INFINITY;   // kind 2: a group's largest score
    }
    unsigned kept[(kRouteMaxGroups + 31) / 32] = {0u, 0u};   // bit `lane` of word i: group lane + 32 i is kept
    for (int pick = 0; pick < keep; ++pick) {
      float best = -INFINITY;
      int arg = 0x7fffffff;
#pragma unroll
      for (int i = 0; i < (kRouteMaxGroups + 31) / 32; ++i) {
        const int g = lane + 32 * i;
        if (g < groups && !(kept[i] & 1u) && (gs[i] > best || (gs[i] == best && g < arg))) best = gs[i], arg = g;
      }
      if (arg == 0x7fffffff) arg = 0x7ffffffe;       // nothing left on this lane
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
        if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
      }
#pragma unroll
      for (int i = 0; i < (kRouteMaxGroups + 31) / 32; ++i)
        if (arg == lane + 32 * i) kept[i] |= 1u;
    }
#pragma unroll
    for (int i = 0; i < (kRouteMaxGroups + 31) / 32; ++i) {
      const int g = lane + 32 * i;
      if (g < groups && !(kept[i] & 1u))
        for (int e = g * per; e < (g + 1) * per; ++e) choice[e] = -INFINITY;
    }
    __syncwarp();
  }
  float wsum = 0.f, mine = 0.f, zmax = 0.f;
  int my_id = 0;
  for (int j = 0; j < top_k; ++j) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float c = choice[e];
      if (c > best || (c == best && e < arg && c > -INFINITY)) best = c, arg = e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) best = ob, arg = oa;
    }
    if (arg >= E) arg = 0;                            // fewer candidates than top_k: cannot happen with keep*per >= top_k
    float s = sg[arg];
    if (kind == 1) {                                 // the first pick is the largest logit
      if (j == 0) zmax = s;
      s = expf(s - zmax);
    }
    wsum += s;
    if (lane == j) mine = s, my_id = arg;
    __syncwarp();
    if (lane == 0) choice[arg] = -INFINITY;
    __syncwarp();
  }
  if (lane < top_k) {
    ids[t * top_k + lane] = my_id;
    weights[t * top_k + lane] = kind == 1 ? mine / wsum : mine / (wsum + 1e-20f) * scale;
  }
}

// ------------------------------------------------------------------ expert GEMMs for any sizes
struct MoeGenericParams {
  const void* a;              // gate_up: x [tokens, K] (row = sorted_pair[pos] / top_k); down: h [pairs, K]
  const void* w;              // gate_up: [E, 2 * n_out, K]; down: [E, n_out, K]
  void* out;                  // gate_up: [pairs, n_out] element type; down: [pairs, n_out] fp32
  const int32_t *offsets, *sorted_pair;
  int64_t a_stride;
  int K, n_out, top_k;
  int act;                    // up alone: 0 silu, 1 relu, 2 gelu (tanh form), 3 squared relu
  float glu_alpha, glu_limit; // gate_up with glu_limit > 0: g sigmoid(alpha g) (u + 1), g = min(gate, limit), u = clamp(up)
};

__device__ __forceinline__ float plain_act(float x, int act) {
  if (act == 1) return fmaxf(x, 0.f);
  if (act == 2) return gelu_tanh_f(x);
  if (act == 3) {
    const float r = fmaxf(x, 0.f);
    return r * r;
  }
  return silu_f(x);
}

constexpr int kGM = 32, kGN = 64, kGK = 16;

// kMode 0: down (fp32 out, rows in plan order); 1: silu(gate) * up; 2: act(up) alone (p.act: the codes of act_only)
template <typename T, int kMode>
__global__ void __launch_bounds__(256)
moe_gemm_generic_kernel(const MoeGenericParams p) {
  constexpr bool kGateUp = kMode == 1;
  constexpr bool kGather = kMode != 0;
  __shared__ float sa[kGK][kGM + 1];
  __shared__ float sb[kGateUp ? 2 : 1][kGK][kGN + 1];
  __shared__ int srow[kGM];
  pdl_wait();
  const int e = blockIdx.z;
  const int row_begin = p.offsets[e], cnt = p.offsets[e + 1] - row_begin;
  if (cnt <= 0) return;
  const int n0 = blockIdx.x * kGN;
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const T* a = reinterpret_cast<const T*>(p.a);
  const T* w = reinterpret_cast<const T*>(p.w) + (int64_t)e * (kGateUp ? 2 : 1) * p.n_out * p.K;
  for (int m0 = blockIdx.y * kGM; m0 < cnt; m0 += gridDim.y * kGM) {
    __syncthreads();
    if (tid < kGM) {
      const int r = m0 + tid;
      srow[tid] = r < cnt ? (kGather ? p.sorted_pair[row_begin + r] / p.top_k : row_begin + r) : -1;
    }
    float acc[2][4], acc2[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f, acc2[i][j] = 0.f;
    for (int k0 = 0; k0 < p.K; k0 += kGK) {
      __syncthreads();
      for (int x = tid; x < kGM * kGK; x += 256) {
        const int r = x / kGK, kk = x % kGK;
        const int src = srow[r];
        sa[kk][r] = (src >= 0 && k0 + kk < p.K) ? to_f32<T>(a[(int64_t)src * p.a_stride + k0 + kk]) : 0.f;
      }
      for (int x = tid; x < kGN * kGK; x += 256) {
        const int c = x / kGK, kk = x % kGK;
        const bool ok = n0 + c < p.n_out && k0 + kk < p.K;
        sb[0][kk][c] = ok ? to_f32<T>(w[(int64_t)(n0 + c) * p.K + k0 + kk]) : 0.f;
        if (kGateUp) sb[1][kk][c] = ok ? to_f32<T>(w[(int64_t)(p.n_out + n0 + c) * p.K + k0 + kk]) : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int kk = 0; kk < kGK; ++kk) {
        const float a0 = sa[kk][ty * 2], a1 = sa[kk][ty * 2 + 1];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float b = sb[0][kk][tx * 4 + j];
          acc[0][j] += a0 * b;
          acc[1][j] += a1 * b;
          if (kGateUp) {
            const float b2 = sb[1][kk][tx * 4 + j];
            acc2[0][j] += a0 * b2;
            acc2[1][j] += a1 * b2;
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int r = m0 + ty * 2 + i;
      if (r >= cnt) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = n0 + tx * 4 + j;
        if (c >= p.n_out) continue;
        const int64_t o = (int64_t)(row_begin + r) * p.n_out + c;
        if (kGateUp) {
          float r;
          if (p.glu_limit > 0.f) {
            const float g = fminf(acc[i][j], p.glu_limit);
            const float u = fminf(fmaxf(acc2[i][j], -p.glu_limit), p.glu_limit);
            r = g * sigmoid_f(p.glu_alpha * g) * (u + 1.0f);
          } else {
            r = silu_f(acc[i][j]) * acc2[i][j];
          }
          reinterpret_cast<T*>(p.out)[o] = from_f32<T>(r);
        }
        else if (kMode == 2) reinterpret_cast<T*>(p.out)[o] = from_f32<T>(plain_act(acc[i][j], p.act));
        else reinterpret_cast<float*>(p.out)[o] = acc[i][j];
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
moe_combine_weighted_kernel(T* __restrict__ out, const float* __restrict__ y, const float* __restrict__ weights,
                            const int32_t* __restrict__ pos_of_pair, int k, int hidden) {
  pdl_wait();
  const int64_t t = blockIdx.x;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < k; ++j) {
      const int ps = pos_of_pair[t * k + j];
      if (ps >= 0) acc += weights[t * k + j] * y[(int64_t)ps * hidden + i];
    }
    out[t * hidden + i] = from_f32<T>(acc);
  }
}

}  // namespace b200

using namespace b200;

extern "C" int b200_moe_route_grouped(int32_t* topk_ids, float* topk_weights, const float* router_logits,
                                      int64_t logit_stride, const float* bias, int32_t tokens,
                                      int32_t num_experts, int32_t top_k, int32_t groups, int32_t keep,
                                      float scale, b200_stream_t stream) {
  B200_RETURN_IF(tokens < 0 || num_experts <= 0 || top_k <= 0 || top_k > num_experts || groups <= 0 || keep <= 0 ||
                     keep > groups || num_experts % groups != 0 || (num_experts / groups) * keep < top_k,
                 B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(num_experts > kRouteMaxExperts || top_k > kRouteMaxTopK || groups > kRouteMaxGroups,
                 B200_ERR_UNSUPPORTED);
  if (tokens == 0) return B200_OK;
  B200_RETURN_IF(!topk_ids || !topk_weights || !router_logits, B200_ERR_NULL_POINTER);
  const size_t smem = (size_t)4 * 2 * num_experts * sizeof(float);
  launch_pdl(moe_route_grouped_kernel, dim3((tokens + 3) / 4), dim3(128), smem, (cudaStream_t)stream, topk_ids,
             topk_weights, router_logits, logit_stride, bias, tokens, num_experts, top_k, groups, keep, scale, 0);
  return finish_launch();
}

extern "C" int b200_moe_route_grouped_softmax(int32_t* topk_ids, float* topk_weights, const float* router_logits,
                                              int64_t logit_stride, int32_t tokens, int32_t num_experts,
                                              int32_t top_k, int32_t groups, int32_t keep, float scale,
                                              b200_stream_t stream) {
  B200_RETURN_IF(tokens < 0 || num_experts <= 0 || top_k <= 0 || top_k > num_experts || groups <= 0 || keep <= 0 ||
                     keep > groups || num_experts % groups != 0 || (num_experts / groups) * keep < top_k,
                 B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(num_experts > kRouteMaxExperts || top_k > kRouteMaxTopK || groups > kRouteMaxGroups,
                 B200_ERR_UNSUPPORTED);
  if (tokens == 0) return B200_OK;
  B200_RETURN_IF(!topk_ids || !topk_weights || !router_logits, B200_ERR_NULL_POINTER);
  const size_t smem = (size_t)4 * 2 * num_experts * sizeof(float);
  launch_pdl(moe_route_grouped_kernel, dim3((tokens + 3) / 4), dim3(128), smem, (cudaStream_t)stream, topk_ids,
             topk_weights, router_logits, logit_stride, (const float*)nullptr, tokens, num_experts, top_k, groups, keep,
             scale, 2);
  return finish_launch();
}

extern "C" int b200_moe_route_topk(int32_t* topk_ids, float* topk_weights, const float* router_logits,
                                   int64_t logit_stride, const float* bias, int32_t tokens, int32_t num_experts,
                                   int32_t top_k, b200_stream_t stream) {
  B200_RETURN_IF(tokens < 0 || num_experts <= 0 || top_k <= 0 || top_k > num_experts, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(num_experts > kRouteMaxExperts || top_k > kRouteMaxTopK, B200_ERR_UNSUPPORTED);
  if (tokens == 0) return B200_OK;
  B200_RETURN_IF(!topk_ids || !topk_weights || !router_logits, B200_ERR_NULL_POINTER);
  const size_t smem = (size_t)4 * 2 * num_experts * sizeof(float);
  launch_pdl(moe_route_grouped_kernel, dim3((tokens + 3) / 4), dim3(128), smem, (cudaStream_t)stream, topk_ids,
             topk_weights, router_logits, logit_stride, bias, tokens, num_experts, top_k, 1, 1, 1.0f, 1);
  return finish_launch();
}

extern "C" int b200_moe_gemm_generic(void* out, const void* a, int64_t a_stride, const void* w,
                                     const int32_t* offsets, const int32_t* sorted_pair, int32_t num_pairs,
                                     int32_t K, int32_t n_out, int32_t num_local, int32_t top_k, int32_t gate_up,
                                     float glu_alpha, float glu_limit, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(num_pairs < 0 || K <= 0 || n_out <= 0 || num_local <= 0 || top_k <= 0, B200_ERR_BAD_SHAPE);
  B200_RETURN_IF(num_local > 65535, B200_ERR_UNSUPPORTED);
  if (num_pairs == 0) return B200_OK;
  B200_RETURN_IF(!out || !a || !w || !offsets || !sorted_pair, B200_ERR_NULL_POINTER);
  B200_RETURN_IF(gate_up < 0 || gate_up > 5, B200_ERR_BAD_SHAPE);
  MoeGenericParams p{a, w, out, offsets, sorted_pair, a_stride, K, n_out, top_k, gate_up >= 2 ? gate_up - 2 : 0,
                     glu_alpha, glu_limit};
  int my = (num_pairs + kGM - 1) / kGM;
  if (my > 32) my = 32;
  const dim3 grid((n_out + kGN - 1) / kGN, my, num_local);
  B200_DISPATCH_3(dtype, T, {
    if (gate_up == 1) launch_pdl(moe_gemm_generic_kernel<T, 1>, grid, dim3(256), 0, (cudaStream_t)stream, p);
    else if (gate_up >= 2) launch_pdl(moe_gemm_generic_kernel<T, 2>, grid, dim3(256), 0, (cudaStream_t)stream, p);
    else launch_pdl(moe_gemm_generic_kernel<T, 0>, grid, dim3(256), 0, (cudaStream_t)stream, p);
  });
  return finish_launch();
}

extern "C" int b200_moe_combine_weighted(void* out, const float* y, const float* topk_weights,
                                         const int32_t* pos_of_pair, int32_t tokens, int32_t top_k,
                                         int32_t hidden, int32_t dtype, b200_stream_t stream) {
  B200_RETURN_IF(tokens < 0 || top_k <= 0 || hidden <= 0, B200_ERR_BAD_SHAPE);
  if (tokens == 0) return B200_OK;
  B200_RETURN_IF(!out || !y || !topk_weights || !pos_of_pair, B200_ERR_NULL_POINTER);
  B200_DISPATCH_3(dtype, T, launch_pdl(moe_combine_weighted_kernel<T>, dim3(tokens), dim3(256), 0, (cudaStream_t)stream,
                                       (T*)out, y, topk_weights, pos_of_pair, top_k, hidden));
  return finish_launch();
}
