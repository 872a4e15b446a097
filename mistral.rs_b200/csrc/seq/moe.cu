// moe.cu — mixture of experts: the routing rule (softmax or sigmoid scores, a choice bias that does not enter the weights,
// selection limited to the best groups of neighbouring experts, a group scored by its largest choice or by the sum of its
// few largest), the expert feed-forward for small batches as two
// weight-streaming kernels, and the sort / gather / combine steps around per-expert matrix products for large ones.
#include "seq_common.cuh"

namespace seq {

constexpr int ROUTE_MAX_EXPERTS = 1024;

// one warp per token; scores and choices of all experts in shared memory
__global__ void moe_route_kernel(const float *__restrict__ logits, const float *__restrict__ correction, int n_tok, int n_experts,
                                 int n_groups, int keep_groups, int top, int renorm, int score_fn, int group_top, float weight_scale,
                                 int32_t *__restrict__ experts, float *__restrict__ weights) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int t = blockIdx.x * nw + wib;
  if (t >= n_tok) return;
  float *score = sm + (size_t)wib * (2 * n_experts + n_groups), *choice = score + n_experts, *gscore = choice + n_experts;
  const float *z = logits + (int64_t)t * n_experts;
  float inv = 1.0f;
  if (score_fn == MRS_SEQ_SCORE_SIGMOID) {
    for (int e = lane; e < n_experts; e += 32) score[e] = sigmoid_f(z[e]);
  } else {
    float mx = -INFINITY;
    for (int e = lane; e < n_experts; e += 32) mx = fmaxf(mx, z[e]);
    mx = warp_max(mx);
    float sum = 0.0f;
    for (int e = lane; e < n_experts; e += 32) {
      const float p = expf(z[e] - mx);
      score[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    inv = 1.0f / sum;
  }
  for (int e = lane; e < n_experts; e += 32) {
    const float s = score[e] * inv;
    score[e] = s;
    choice[e] = s + (correction ? correction[e] : 0.0f);
  }
  __syncwarp();
  const int per = n_experts / n_groups;
  if (keep_groups < n_groups) {
    for (int gi = lane; gi < n_groups; gi += 32) {
      float best = -INFINITY;
      if (group_top <= 1) {
        for (int e = gi * per; e < (gi + 1) * per; e++) best = fmaxf(best, choice[e]);
      } else {      // the sum of the group's group_top largest choices: take them one by one, below the last one taken
        float total = 0.0f, last = INFINITY;
        int last_e = -1;
        for (int r = 0; r < group_top && r < per; r++) {
          float bv = -INFINITY;
          int be = -1;
          for (int e = gi * per; e < (gi + 1) * per; e++) {
            const float v = choice[e];
            if ((v < last || (v == last && e > last_e)) && (be < 0 || v > bv)) { bv = v; be = e; }
          }
          if (be < 0) break;
          total += bv;
          last = bv;
          last_e = be;
        }
        best = total;
      }
      gscore[gi] = best;
    }
    __syncwarp();
    // take the keep_groups best groups one by one (ties: the lower index); a taken group is marked with +inf
    for (int r = 0; r < keep_groups; r++) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int gi = lane; gi < n_groups; gi += 32) {
        const float v = gscore[gi];
        if (v != INFINITY && (v > bv || (v == bv && gi < bi))) { bv = v; bi = gi; }
      }
      for (int m = 16; m > 0; m >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
      }
      if (lane == 0 && bi < n_groups) gscore[bi] = INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < n_experts; e += 32)
      if (gscore[e / per] != INFINITY) choice[e] = -INFINITY;
    __syncwarp();
  }
  float wsum = 0.0f;
  for (int r = 0; r < top; r++) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = choice[e];
      if (!(v != v) && (v > bv || (v == bv && e < bi)) && v != -INFINITY) { bv = v; bi = e; }
    }
    for (int m = 16; m > 0; m >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) bi = 0;   // fewer eligible experts than `top`: weight 0
    const float wv = bv == -INFINITY ? 0.0f : score[bi];
    if (lane == 0) {
      experts[(int64_t)t * top + r] = bi;
      weights[(int64_t)t * top + r] = wv;
      if (bv != -INFINITY) choice[bi] = -INFINITY;
    }
    wsum += wv;
    __syncwarp();
  }
  if (renorm && lane == 0 && wsum > 0.0f)
    for (int r = 0; r < top; r++) weights[(int64_t)t * top + r] /= wsum;
  if (weight_scale != 1.0f && lane == 0)
    for (int r = 0; r < top; r++) weights[(int64_t)t * top + r] *= weight_scale;
}

// hidden[t][k][r] = act(gate_up[e][r] . x_t) * (gate_up[e][ff + r] . x_t): one warp per output element;
// blockIdx.y is the (token, k) pair, pairs laid out [token][k]
template <typename T>
__global__ void __launch_bounds__(256) moe_gate_up_kernel(const T *__restrict__ x, const T *__restrict__ gate_up,
                                                          const int32_t *__restrict__ experts, int top, int width, int ff,
                                                          const mrs_seq_glu_rule rule, T *__restrict__ hidden) {
  extern __shared__ __align__(16) float xs[];   // [width]
  const int pair = blockIdx.y, tok = pair / top;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int e = experts[pair];
  for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32<T>(x[(int64_t)tok * width + c]);
  __syncthreads();
  const T *w = gate_up + (int64_t)e * 2 * ff * width;
  const bool vec = width % Vec16<T>::N == 0 && ((uintptr_t)gate_up % 16) == 0;
  for (int r = blockIdx.x * nw + wib; r < ff; r += gridDim.x * nw) {
    const float ag = warp_row_dot<T>(w + (int64_t)r * width, xs, width, lane, vec);
    const float au = warp_row_dot<T>(w + (int64_t)(ff + r) * width, xs, width, lane, vec);
    if (lane == 0) {
      // the products leave the "matrix product" in the activation type, as the large-batch path's do
      const float gt = to_f32<T>(from_f32<T>(ag)), up = to_f32<T>(from_f32<T>(au));
      hidden[(int64_t)pair * ff + r] = from_f32<T>(glu_join(gt, up, rule));
    }
  }
}

// the plain rule, one warp per token: the `top` largest logits (ties: the lower index), softmax over those alone
__global__ void moe_route_top_softmax_kernel(const float *__restrict__ logits, int n_tok, int n_experts, int top,
                                             int32_t *__restrict__ experts, float *__restrict__ weights) {
  extern __shared__ float sm[];
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int t = blockIdx.x * nw + wib;
  if (t >= n_tok) return;
  float *z = sm + (size_t)wib * n_experts;
  for (int e = lane; e < n_experts; e += 32) z[e] = logits[(int64_t)t * n_experts + e];
  __syncwarp();
  float first = 0.0f, sum = 0.0f;
  for (int r = 0; r < top; r++) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < n_experts; e += 32) {
      const float v = z[e];
      if (v == v && (bi == 0x7fffffff ? v >= bv : v > bv)) { bv = v; bi = e; }   // NaN never wins; a taken expert holds NaN
    }
    for (int m = 16; m > 0; m >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, m);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    if (bi == 0x7fffffff) { bi = 0; bv = -INFINITY; }
    if (r == 0) first = bv;                       // the largest logit: the softmax's reference point
    const float p = expf(bv - first);
    sum += p;
    if (lane == 0) {
      experts[(int64_t)t * top + r] = bi;
      weights[(int64_t)t * top + r] = p;
      z[bi] = __int_as_float(0x7fc00000);
    }
    __syncwarp();
  }
  if (lane == 0)
    for (int r = 0; r < top; r++) weights[(int64_t)t * top + r] /= sum;
}

// hidden[t][k][r] = act(up[e][r] . x_t): experts without a gate; the layout of moe_gate_up_kernel
template <typename T>
__global__ void __launch_bounds__(256) moe_up_kernel(const T *__restrict__ x, const T *__restrict__ up, const int32_t *__restrict__ experts,
                                                     int top, int width, int ff, int act, T *__restrict__ hidden) {
  extern __shared__ __align__(16) float xs[];   // [width]
  const int pair = blockIdx.y, tok = pair / top;
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int e = experts[pair];
  for (int c = threadIdx.x; c < width; c += blockDim.x) xs[c] = to_f32<T>(x[(int64_t)tok * width + c]);
  __syncthreads();
  const T *w = up + (int64_t)e * ff * width;
  const bool vec = width % Vec16<T>::N == 0 && ((uintptr_t)up % 16) == 0;
  for (int r = blockIdx.x * nw + wib; r < ff; r += gridDim.x * nw) {
    const float a = warp_row_dot<T>(w + (int64_t)r * width, xs, width, lane, vec);
    if (lane == 0) hidden[(int64_t)pair * ff + r] = from_f32<T>(apply_act(to_f32<T>(from_f32<T>(a)), act));
  }
}

// out[t][r] = sum_k weights[t][k] * (down[e_k][r] . hidden[t][k])
template <typename T>
__global__ void __launch_bounds__(256) moe_down_kernel(const T *__restrict__ hidden, const T *__restrict__ down,
                                                       const int32_t *__restrict__ experts, const float *__restrict__ weights, int top,
                                                       int width, int ff, T *__restrict__ out) {
  extern __shared__ __align__(16) float hs[];   // [top][ff]
  const int t = blockIdx.y, lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int c = threadIdx.x; c < top * ff; c += blockDim.x) hs[c] = to_f32<T>(hidden[(int64_t)t * top * ff + c]);
  __syncthreads();
  const bool vec = ff % Vec16<T>::N == 0 && ((uintptr_t)down % 16) == 0;
  for (int r = blockIdx.x * nw + wib; r < width; r += gridDim.x * nw) {
    float acc = 0.0f;
    for (int k = 0; k < top; k++) {
      const T *wd = down + ((int64_t)experts[(int64_t)t * top + k] * width + r) * ff;
      const float a = warp_row_dot<T>(wd, hs + k * ff, ff, lane, vec);
      acc = fmaf(weights[(int64_t)t * top + k], to_f32<T>(from_f32<T>(a)), acc);
    }
    if (lane == 0) out[(int64_t)t * width + r] = from_f32<T>(acc);
  }
}

// ---- sorted path --------------------------------------------------------------------------------------------------
// single CTA: counts per expert, then every (token, k) pair takes the next free row of its expert's range
__global__ void moe_sort_kernel(const int32_t *__restrict__ experts, int n_pairs, int n_experts, int32_t *__restrict__ counts,
                                int32_t *__restrict__ order) {
  extern __shared__ int32_t cnt[];   // [n_experts] counts, then [n_experts] running offsets
  int32_t *off = cnt + n_experts;
  for (int e = threadIdx.x; e < n_experts; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) atomicAdd(&cnt[experts[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < n_experts; e++) {
      off[e] = run;
      run += cnt[e];
      counts[e] = cnt[e];
    }
  }
  __syncthreads();
  // rows of one expert may land in any order: each row's product does not depend on its place
  for (int i = threadIdx.x; i < n_pairs; i += blockDim.x) order[atomicAdd(&off[experts[i]], 1)] = i;
}

template <typename T>
__global__ void moe_gather_kernel(const T *__restrict__ x, const int32_t *__restrict__ order, int top, int width, T *__restrict__ sorted) {
  const int i = blockIdx.x, t = order[i] / top;
  for (int c = threadIdx.x; c < width; c += blockDim.x) sorted[(int64_t)i * width + c] = x[(int64_t)t * width + c];
}

__global__ void moe_inverse_kernel(const int32_t *__restrict__ order, int n_pairs, int32_t *__restrict__ inverse) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_pairs) inverse[order[i]] = i;
}

template <typename T>
__global__ void moe_combine_kernel(const T *__restrict__ sorted_y, const int32_t *__restrict__ inverse, const float *__restrict__ weights,
                                   int top, int width, T *__restrict__ out) {
  const int t = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float acc = 0.0f;
    for (int k = 0; k < top; k++)
      acc = fmaf(weights[(int64_t)t * top + k], to_f32<T>(sorted_y[(int64_t)inverse[(int64_t)t * top + k] * width + c]), acc);
    out[(int64_t)t * width + c] = from_f32<T>(acc);
  }
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_moe_route(const float *logits, const float *correction, int n_tok, int n_experts, int n_groups, int keep_groups,
                                 int top, int renorm, int32_t *experts, float *weights, int64_t stream) {
  return mrs_seq_moe_route_scored(logits, correction, n_tok, n_experts, n_groups, keep_groups, top, renorm, MRS_SEQ_SCORE_SOFTMAX, 1, 1.0f,
                                  experts, weights, stream);
}

extern "C" int mrs_seq_moe_route_scored(const float *logits, const float *correction, int n_tok, int n_experts, int n_groups, int keep_groups,
                                        int top, int renorm, int score_fn, int group_top, float weight_scale, int32_t *experts,
                                        float *weights, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (n_experts < 1 || n_experts > ROUTE_MAX_EXPERTS || n_groups < 1 || n_experts % n_groups || keep_groups < 1 ||
      keep_groups > n_groups || top < 1 || top > n_experts || group_top < 1 ||
      (score_fn != MRS_SEQ_SCORE_SOFTMAX && score_fn != MRS_SEQ_SCORE_SIGMOID))
    return -2;
  const int warps = 4;
  const size_t bytes = (size_t)warps * (2 * n_experts + n_groups) * sizeof(float);
  moe_route_kernel<<<(n_tok + warps - 1) / warps, warps * 32, bytes, (cudaStream_t)stream>>>(
      logits, correction, n_tok, n_experts, n_groups, keep_groups, top, renorm, score_fn, group_top, weight_scale, experts, weights);
  return launch_status();
}

extern "C" int mrs_seq_moe_route_top_softmax(const float *logits, int n_tok, int n_experts, int top, int32_t *experts, float *weights,
                                             int64_t stream) {
  if (n_tok <= 0) return 0;
  if (n_experts < 1 || n_experts > ROUTE_MAX_EXPERTS || top < 1 || top > n_experts) return -2;
  const int warps = 4;
  moe_route_top_softmax_kernel<<<(n_tok + warps - 1) / warps, warps * 32, (size_t)warps * n_experts * sizeof(float), (cudaStream_t)stream>>>(
      logits, n_tok, n_experts, top, experts, weights);
  return launch_status();
}

extern "C" int mrs_seq_moe_up(const void *x, const void *up, int dtype, const int32_t *experts, int n_tok, int top, int width, int ff,
                              int act, void *hidden, int64_t stream) {
  if (n_tok <= 0) return 0;
  if ((size_t)width * sizeof(float) > 160 * 1024) return -2;
  const int warps = 8, bx = (ff + warps - 1) / warps;
  const size_t bytes = (size_t)width * sizeof(float);
  SEQ_DISPATCH_DTYPE(dtype, {
    auto kern = moe_up_kernel<T>;
    static size_t allowed = 48 * 1024;
    if (bytes > allowed) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
      allowed = bytes;
    }
    kern<<<dim3(bx < 256 ? bx : 256, n_tok * top), warps * 32, bytes, (cudaStream_t)stream>>>((const T *)x, (const T *)up, experts, top, width,
                                                                                             ff, act, (T *)hidden);
  });
  return launch_status();
}

extern "C" int mrs_seq_moe_gate_up(const void *x, const void *gate_up, int dtype, const int32_t *experts, int n_tok, int top, int width,
                                   int ff, int act, void *hidden, int64_t stream) {
  const mrs_seq_glu_rule rule = {act, 0.0f, 0.0f, 0.0f};
  return mrs_seq_moe_gate_up_rule(x, gate_up, dtype, experts, n_tok, top, width, ff, &rule, hidden, stream);
}

extern "C" int mrs_seq_moe_gate_up_rule(const void *x, const void *gate_up, int dtype, const int32_t *experts, int n_tok, int top, int width,
                                        int ff, const mrs_seq_glu_rule *rule, void *hidden, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (!rule) return -2;
  if ((size_t)width * sizeof(float) > 160 * 1024) return -2;
  const int warps = 8, bx = (ff + warps - 1) / warps;
  const size_t bytes = (size_t)width * sizeof(float);
  SEQ_DISPATCH_DTYPE(dtype, {
    auto kern = moe_gate_up_kernel<T>;
    static size_t allowed = 48 * 1024;
    if (bytes > allowed) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
      allowed = bytes;
    }
    kern<<<dim3(bx < 256 ? bx : 256, n_tok * top), warps * 32, bytes, (cudaStream_t)stream>>>(
        (const T *)x, (const T *)gate_up, experts, top, width, ff, *rule, (T *)hidden);
  });
  return launch_status();
}

extern "C" int mrs_seq_moe_down(const void *hidden, const void *down, int dtype, const int32_t *experts, const float *weights, int n_tok,
                                int top, int width, int ff, void *out, int64_t stream) {
  if (n_tok <= 0) return 0;
  const size_t bytes = (size_t)top * ff * sizeof(float);
  if (bytes > 160 * 1024) return -2;
  const int warps = 8, bx = (width + warps - 1) / warps;
  SEQ_DISPATCH_DTYPE(dtype, {
    auto kern = moe_down_kernel<T>;
    static size_t allowed = 48 * 1024;
    if (bytes > allowed) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
      allowed = bytes;
    }
    kern<<<dim3(bx < 256 ? bx : 256, n_tok), warps * 32, bytes, (cudaStream_t)stream>>>(
        (const T *)hidden, (const T *)down, experts, weights, top, width, ff, (T *)out);
  });
  return launch_status();
}

extern "C" int mrs_seq_moe_sort(const int32_t *experts, int n_pairs, int n_experts, int32_t *counts, int32_t *order, int64_t stream) {
  if (n_pairs <= 0) return 0;
  moe_sort_kernel<<<1, 1024, 2 * n_experts * sizeof(int32_t), (cudaStream_t)stream>>>(experts, n_pairs, n_experts, counts, order);
  return launch_status();
}

extern "C" int mrs_seq_moe_gather(const void *x, int dtype, const int32_t *order, int n_pairs, int top, int width, void *sorted,
                                  int64_t stream) {
  if (n_pairs <= 0) return 0;
  SEQ_DISPATCH_DTYPE(dtype, (moe_gather_kernel<T><<<n_pairs, 128, 0, (cudaStream_t)stream>>>((const T *)x, order, top, width, (T *)sorted)));
  return launch_status();
}

extern "C" int mrs_seq_moe_combine(const void *sorted_y, int dtype, const int32_t *order, const float *weights, int n_tok, int top,
                                   int width, int32_t *scratch_inverse, void *out, int64_t stream) {
  if (n_tok <= 0) return 0;
  const int n_pairs = n_tok * top;
  moe_inverse_kernel<<<(n_pairs + 255) / 256, 256, 0, (cudaStream_t)stream>>>(order, n_pairs, scratch_inverse);
  SEQ_DISPATCH_DTYPE(dtype, (moe_combine_kernel<T><<<n_tok, 128, 0, (cudaStream_t)stream>>>((const T *)sorted_y, scratch_inverse, weights,
                                                                                          top, width, (T *)out)));
  return launch_status();
}
