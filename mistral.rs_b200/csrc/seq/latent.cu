// latent.cu — attention whose keys and values are decompressed from one small latent per token (multi-head latent
// attention): the cache holds, per token, the normed latent c [kv_rank] followed by one rotated key part [rot_dim] that
// all heads share.  Because k_h = W_uk,h c and v_h = W_uv,h c are linear in c, a head's score is
// (W_uk,h^T q_h) . c + q_rot,h . k_rot and its output W_uv,h (sum_j p_j c_j): attention runs over the latent rows
// themselves as ONE key/value head of size kv_rank + rot_dim whose values are the first kv_rank columns of the keys
// (the paged kernels of window_attn.cu with row strides, or the tensor-core kernel of latent_attn_mma.cu).  This file
// holds what surrounds the matrix products: the latent norms, the rotation in neighbouring pairs and the cache write.
#include "seq_common.cuh"

namespace seq {

// One CTA per token.  Warp 0.. split the work by parts: the query latent's norm, the key/value latent's norm + store, the
// shared key part's rotation + store.  Sums of squares go through the block.
template <typename T>
__global__ void __launch_bounds__(256) latent_prepare_kernel(const mrs_seq_latent_prepare_args a) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const T *y = (const T *)a.y + (int64_t)t * a.y_ld;
  if (a.q_rank > 0) {
    const T *src = y + a.q_col;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < a.q_rank; c += blockDim.x) {
      const float v = to_f32<T>(src[c]);
      ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf_exact(block_sum(ss, red) / (float)a.q_rank + a.eps);
    T *dst = (T *)a.q_out + (int64_t)t * a.q_out_ld;
    for (int c = threadIdx.x; c < a.q_rank; c += blockDim.x) dst[c] = from_f32<T>(to_f32<T>(src[c]) * inv * a.q_norm_w[c]);
  }
  if (a.kv_rank <= 0) return;
  const int64_t slot = a.slot_of_tok[t];
  if (slot < 0) return;       // uniform over the block
  const T *src = y + a.kv_col;
  T *dst = (T *)a.cache + slot * a.cache_row;
  float ss = 0.0f;
  for (int c = threadIdx.x; c < a.kv_rank; c += blockDim.x) {
    const float v = to_f32<T>(src[c]);
    ss = fmaf(v, v, ss);
  }
  const float inv = rsqrtf_exact(block_sum(ss, red) / (float)a.kv_rank + a.eps);
  T *dense = a.kv_out ? (T *)a.kv_out + (int64_t)t * a.kv_out_ld : nullptr;      // the normed latent also as a dense row of the step
  for (int c = threadIdx.x; c < a.kv_rank; c += blockDim.x) {
    const T r = from_f32<T>(to_f32<T>(src[c]) * inv * a.kv_norm_w[c]);
    dst[c] = r;
    if (dense) dense[c] = r;
  }
  const int half = a.cos_sin ? a.rot_dims / 2 : 0;
  const float2 *cs = (const float2 *)a.cos_sin + (int64_t)t * half;
  src += a.kv_rank;
  dst += a.kv_rank;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float u = to_f32<T>(src[2 * i]), v = to_f32<T>(src[2 * i + 1]);
    const float2 c = cs[i];
    dst[2 * i] = from_f32<T>(u * c.x - v * c.y);
    dst[2 * i + 1] = from_f32<T>(v * c.x + u * c.y);
  }
  for (int d = 2 * half + threadIdx.x; d < a.rot_dim; d += blockDim.x) dst[d] = src[d];
}

// one CTA per token, all heads: out[t][h][:dims] = in[t][h][:dims] with the first rot_dims entries turned in neighbouring pairs
template <typename T>
__global__ void rotate_pairs_kernel(const T *__restrict__ in, int64_t in_ld, int64_t in_head, T *__restrict__ out, int64_t out_ld,
                                    int64_t out_head, int heads, int dims, int rot_dims, const float2 *__restrict__ cos_sin) {
  const int t = blockIdx.x, half = cos_sin ? rot_dims / 2 : 0, pairs = dims / 2;
  const T *src = in + (int64_t)t * in_ld;
  T *dst = out + (int64_t)t * out_ld;
  const float2 *cs = cos_sin + (int64_t)t * half;
  for (int e = threadIdx.x; e < heads * pairs; e += blockDim.x) {
    const int h = e / pairs, i = e % pairs;
    const T *s = src + (int64_t)h * in_head + 2 * i;
    T *d = dst + (int64_t)h * out_head + 2 * i;
    if (i < half) {
      const float u = to_f32<T>(s[0]), v = to_f32<T>(s[1]);
      const float2 c = cs[i];
      d[0] = from_f32<T>(u * c.x - v * c.y);
      d[1] = from_f32<T>(v * c.x + u * c.y);
    } else {
      d[0] = s[0];
      d[1] = s[1];
    }
  }
  if (dims & 1)
    for (int h = threadIdx.x; h < heads; h += blockDim.x) dst[(int64_t)h * out_head + dims - 1] = src[(int64_t)h * in_head + dims - 1];
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_latent_prepare(const mrs_seq_latent_prepare_args *args, int64_t stream) {
  const mrs_seq_latent_prepare_args &a = *args;
  if (a.n_tok <= 0) return 0;
  if (!a.y || a.q_rank < 0 || a.kv_rank < 0 || (a.q_rank == 0 && a.kv_rank == 0)) return -2;
  if (a.q_rank > 0 && (!a.q_norm_w || !a.q_out)) return -2;
  if (a.kv_rank > 0 && (!a.kv_norm_w || !a.cache || !a.slot_of_tok || a.rot_dim < 0 || a.cache_row < a.kv_rank + a.rot_dim)) return -2;
  if (a.kv_rank > 0 && a.cos_sin && (a.rot_dims < 2 || a.rot_dims % 2 || a.rot_dims > a.rot_dim)) return -2;
  const int widest = a.q_rank > a.kv_rank ? a.q_rank : a.kv_rank;
  const int th = widest >= 1024 ? 256 : (widest >= 256 ? 128 : 64);
  SEQ_DISPATCH_DTYPE(a.dtype, (latent_prepare_kernel<T><<<a.n_tok, th, 0, (cudaStream_t)stream>>>(a)));
  return launch_status();
}

extern "C" int mrs_seq_rotate_pairs(const void *in, int64_t in_ld, int64_t in_head, void *out, int64_t out_ld, int64_t out_head, int dtype,
                                    int heads, int dims, int rot_dims, const float *cos_sin, int n_tok, int64_t stream) {
  if (n_tok <= 0 || heads <= 0 || dims <= 0) return 0;
  if (cos_sin && (rot_dims < 2 || rot_dims % 2 || rot_dims > dims)) return -2;
  const int items = heads * (dims / 2), th = items >= 256 ? 256 : (items >= 128 ? 128 : 64);
  SEQ_DISPATCH_DTYPE(dtype, (rotate_pairs_kernel<T><<<n_tok, th, 0, (cudaStream_t)stream>>>(
                                (const T *)in, in_ld, in_head, (T *)out, out_ld, out_head, heads, dims, rot_dims, (const float2 *)cos_sin)));
  return launch_status();
}
