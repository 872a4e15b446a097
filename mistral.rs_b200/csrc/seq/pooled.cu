// pooled.cu — what surrounds softmax attention whose far past is seen in averaged blocks and whose weights are mixed across
// heads:
//   * pool_blocks: when a step stores the last position of a block of `pool` positions, the mean of the block's cached keys
//     and of its cached values is written to the block's own cache row (behind the token rows; window_attn.cu's key_row has
//     the layout).  The attention kernel then reads, for a query, the averaged rows of the blocks that lie wholly before its
//     window and the single rows of the window itself, under one softmax.
//   * mix_heads: weights mixed after the softmax, w'_h = sum_g M[h][g] w_g, applied by head h to the values of its own
//     key/value head.  By linearity out_h = sum_g M[h][g] (w_g applied to the values of h's key/value head): the attention
//     kernel applies every head's weights to ALL value heads (f32), this kernel takes the weighted sum over g and applies the
//     output gate.
//   * gate_cols: an output gate per entry or per head on rows of the activation type.
#include "seq_common.cuh"

namespace seq {

// one CTA per token; only a token whose position ends a block works.  The block's rows were stored by this or an earlier
// step and are read through the page table; sum in f32 in position order, divided by the block size.
template <typename T>
__global__ void pool_blocks_kernel(T *__restrict__ k_cache, T *__restrict__ v_cache, int64_t k_row, int64_t v_row, int k_cols, int v_cols,
                                   int pool, int64_t pool_base, const int32_t *__restrict__ pages, int pages_ld, int page_size,
                                   const int32_t *__restrict__ seq_of_tok, const int32_t *__restrict__ pos_of_tok) {
  const int t = blockIdx.x, pos = pos_of_tok[t];
  if ((pos + 1) % pool != 0) return;
  const int b = (pos + 1) / pool - 1, p0 = b * pool;
  const int32_t *table = pages + (int64_t)seq_of_tok[t] * pages_ld;
  const int per_page = (page_size + pool - 1) / pool, page = p0 / page_size, first = (page * page_size + pool - 1) / pool;
  const int64_t dst = pool_base + (int64_t)table[page] * per_page + (b - first);
  const float n = (float)pool;
  for (int c = threadIdx.x; c < k_cols + v_cols; c += blockDim.x) {
    const bool is_k = c < k_cols;
    T *cache = is_k ? k_cache : v_cache;
    const int64_t ld = is_k ? k_row : v_row;
    const int col = is_k ? c : c - k_cols;
    float s = 0.0f;
    for (int r = 0; r < pool; r++) {
      const int p = p0 + r;
      s += to_f32<T>(cache[((int64_t)table[p / page_size] * page_size + p % page_size) * ld + col]);
    }
    cache[dst * ld + col] = from_f32<T>(s / n);
  }
}

// one CTA per token; a thread takes VEC neighbouring entries of one head (16-byte loads of the f32 rows when VEC is 4); the
// mixing matrix sits in shared memory, the token's `a` rows come through L1
template <typename T, int VEC>
__global__ void mix_heads_kernel(const float *__restrict__ a, const float *__restrict__ mix, const T *__restrict__ gate, int64_t gate_ld,
                                 int gate_act, T *__restrict__ out, int64_t out_ld, int heads, int kv_heads, int dv) {
  extern __shared__ float m[];      // [heads][heads]
  for (int e = threadIdx.x; e < heads * heads; e += blockDim.x) m[e] = mix[e];
  __syncthreads();
  const int t = blockIdx.x, all = kv_heads * dv, per = heads / kv_heads;
  const float *at = a + (int64_t)t * heads * all;
  for (int e = threadIdx.x * VEC; e < heads * dv; e += blockDim.x * VEC) {
    const int h = e / dv, d = e % dv, col = (h / per) * dv + d;
    float s[VEC];
#pragma unroll
    for (int x = 0; x < VEC; x++) s[x] = 0.0f;
    for (int g = 0; g < heads; g++) {
      const float w = m[h * heads + g];
      if (VEC == 4) {
        const float4 v = *(const float4 *)(at + (int64_t)g * all + col);
        s[0] = fmaf(w, v.x, s[0]); s[1 % VEC] = fmaf(w, v.y, s[1 % VEC]); s[2 % VEC] = fmaf(w, v.z, s[2 % VEC]); s[3 % VEC] = fmaf(w, v.w, s[3 % VEC]);
      } else {
        s[0] = fmaf(w, at[(int64_t)g * all + col], s[0]);
      }
    }
    if (gate) {
      if (VEC == 4) {
        const float4 gv = act4(load4<T>(gate + (int64_t)t * gate_ld + e), gate_act);
        s[0] *= gv.x; s[1 % VEC] *= gv.y; s[2 % VEC] *= gv.z; s[3 % VEC] *= gv.w;
      } else {
        s[0] *= apply_act(to_f32<T>(gate[(int64_t)t * gate_ld + e]), gate_act);
      }
    }
    if (VEC == 4) store4<T>(out + (int64_t)t * out_ld + e, make_float4(s[0], s[1 % VEC], s[2 % VEC], s[3 % VEC]));
    else out[(int64_t)t * out_ld + e] = from_f32<T>(s[0]);
  }
}

template <typename T>
__global__ void gate_cols_kernel(T *__restrict__ x, int64_t x_ld, const T *__restrict__ gate, int64_t gate_ld, int cols, int group, int act) {
  const int t = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < cols; c += gridDim.y * blockDim.x) {
    const float g = apply_act(to_f32<T>(gate[(int64_t)t * gate_ld + c / group]), act);
    x[(int64_t)t * x_ld + c] = from_f32<T>(to_f32<T>(x[(int64_t)t * x_ld + c]) * g);
  }
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_pool_blocks(void *k_cache, void *v_cache, int dtype, int64_t k_row, int64_t v_row, int k_cols, int v_cols, int pool,
                                   int64_t pool_base, const int32_t *pages, int pages_ld, int page_size, const int32_t *seq_of_tok,
                                   const int32_t *pos_of_tok, int n_tok, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (!k_cache || !v_cache || pool <= 0 || page_size <= 0 || k_cols <= 0 || v_cols <= 0 || k_row < k_cols || v_row < v_cols) return -2;
  const int items = k_cols + v_cols, th = items >= 512 ? 256 : (items >= 128 ? 128 : 64);
  SEQ_DISPATCH_DTYPE(dtype, (pool_blocks_kernel<T><<<n_tok, th, 0, (cudaStream_t)stream>>>((T *)k_cache, (T *)v_cache, k_row, v_row, k_cols, v_cols,
                                                                                         pool, pool_base, pages, pages_ld, page_size,
                                                                                         seq_of_tok, pos_of_tok)));
  return launch_status();
}

extern "C" int mrs_seq_mix_heads(const float *a, const float *mix, const void *gate, int64_t gate_ld, int gate_act, void *out, int64_t out_ld,
                                 int dtype, int heads, int kv_heads, int dv, int n_tok, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (!a || !mix || !out || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dv <= 0 || heads > 96) return -2;
  const int elem = dtype == MRS_SEQ_BF16 ? 2 : 4;
  auto al = [](const void *p, int by) { return ((uintptr_t)p % by) == 0; };
  const bool vec = dv % 4 == 0 && al(a, 16) && al(out, 4 * elem) && out_ld % 4 == 0 && (!gate || (al(gate, 4 * elem) && gate_ld % 4 == 0));
  const int items = vec ? heads * dv / 4 : heads * dv, th = items >= 1024 ? 256 : (items >= 256 ? 128 : 64);
  const size_t bytes = (size_t)heads * heads * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
  SEQ_DISPATCH_DTYPE(dtype, {
    if (vec) mix_heads_kernel<T, 4><<<n_tok, th, bytes, st>>>(a, mix, (const T *)gate, gate_ld, gate_act, (T *)out, out_ld, heads, kv_heads, dv);
    else mix_heads_kernel<T, 1><<<n_tok, th, bytes, st>>>(a, mix, (const T *)gate, gate_ld, gate_act, (T *)out, out_ld, heads, kv_heads, dv);
  });
  return launch_status();
}

extern "C" int mrs_seq_gate_cols(void *x, int64_t x_ld, const void *gate, int64_t gate_ld, int dtype, int cols, int group, int act, int n_tok,
                                 int64_t stream) {
  if (n_tok <= 0 || cols <= 0) return 0;
  if (!x || !gate || group <= 0) return -2;
  const int by = (cols + 255) / 256;
  SEQ_DISPATCH_DTYPE(dtype, (gate_cols_kernel<T><<<dim3(n_tok, by < 64 ? by : 64), 256, 0, (cudaStream_t)stream>>>(
                                (T *)x, x_ld, (const T *)gate, gate_ld, cols, group, act)));
  return launch_status();
}
