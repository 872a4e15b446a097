// depth.cu — a single f32 residual with RMS norms whose sublayer outputs are added with a multiplier and whose layers
// hand on a depth-weighted average: what enters layer i + 1 is a learned mix of the embedding output and the results of
// layers 0 .. i (the averaging of DenseFormer-style models), not layer i's result alone.  One kernel per sublayer does
// the residual add, stores the layer's result into the step's history, forms the mix over the history and produces the
// next sublayer's normed input — the fusion the multi-stream kernels (streams.cu) make for hyper-connections.  One CTA
// per token; the token's row stays in shared memory between the passes; the residual never leaves f32.
#include "seq_common.cuh"

namespace seq {

template <typename T>
__global__ void embed_scaled_kernel(const T *__restrict__ table, const int32_t *__restrict__ ids, float scale, float *__restrict__ out,
                                    int width) {
  const int t = blockIdx.x;
  const T *row = table + (int64_t)ids[t] * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[(int64_t)t * width + c] = to_f32<T>(row[c]) * scale;
}

// One CTA per token: the token's embedding row times a scale plus a row of the pair table chosen by a hash of (previous
// token, token).  Inside a portion the previous token is the row before; a portion's first token takes it from the
// sequence's state slot, and that same CTA then leaves the portion's last token there (one reader and writer per slot).
template <typename T>
__global__ void embed_pair_kernel(const T *__restrict__ table, const T *__restrict__ pairs, const int32_t *__restrict__ ids, float scale,
                                  int64_t buckets, int64_t mul_prev, int64_t mul_cur, int32_t *__restrict__ prev_state,
                                  const int32_t *__restrict__ cu_tok, const int32_t *__restrict__ past, const int32_t *__restrict__ slot,
                                  const int32_t *__restrict__ seq_of_tok, float *__restrict__ out, int width) {
  const int t = blockIdx.x, s = seq_of_tok[t], first = cu_tok[s];
  const int64_t id = ids[t];
  int64_t r;
  if (t > first) {
    r = ((int64_t)ids[t - 1] * mul_prev + id * mul_cur) % buckets;
  } else {
    const int sl = slot[s];
    r = past[s] > 0 ? ((int64_t)prev_state[sl] * mul_prev + id * mul_cur) % buckets : buckets;
    __syncthreads();                      // every thread has read the slot before it is rewritten
    if (threadIdx.x == 0) prev_state[sl] = ids[cu_tok[s + 1] - 1];
  }
  if (r < 0) r += buckets;
  const T *row = table + id * width, *extra = pairs + r * width;
  for (int c = threadIdx.x; c < width; c += blockDim.x) out[(int64_t)t * width + c] = fmaf(to_f32<T>(row[c]), scale, to_f32<T>(extra[c]));
}

template <typename T, int VEC>
__global__ void __launch_bounds__(1024) rms_residual_kernel(const mrs_seq_rms_residual_args a) {
  extern __shared__ __align__(16) float row[];   // [width]
  __shared__ float red[33];
  __shared__ float mix[128];
  const int t = blockIdx.x, width = a.width;
  const int64_t at = (int64_t)t * width;
  const T *y = (const T *)a.y;
  const int n_hist = a.hist ? a.n_hist : 0;
  for (int j = threadIdx.x; j < n_hist; j += blockDim.x) mix[j] = a.mix[j];
  __syncthreads();
  float inv_y = 1.0f;
  if (y && a.post_w) {       // the sublayer's output is normed before it is added: its row waits in shared memory as f32
    float sy = 0.0f;
    for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
      float yv[VEC];
      if (VEC == 4) { const float4 q = load4<T>(y + at + c); yv[0] = q.x; yv[1 % VEC] = q.y; yv[2 % VEC] = q.z; yv[3 % VEC] = q.w; }
      else yv[0] = to_f32<T>(y[at + c]);
#pragma unroll
      for (int e = 0; e < VEC; e++) {
        row[c + e] = yv[e];
        sy = fmaf(yv[e], yv[e], sy);
      }
    }
    inv_y = rsqrtf_exact(block_sum(sy, red) / (float)width + a.eps);
  }
  float ss = 0.0f;
  for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {
    float v[VEC];
    if (VEC == 4) { const float4 q = *(const float4 *)(a.src + at + c); v[0] = q.x; v[1 % VEC] = q.y; v[2 % VEC] = q.z; v[3 % VEC] = q.w; }
    else v[0] = a.src[at + c];
    if (y && a.post_w) {     // every thread re-reads the columns it staged itself
#pragma unroll
      for (int e = 0; e < VEC; e++) v[e] = fmaf(a.mult, row[c + e] * inv_y * a.post_w[c + e], v[e]);
    } else if (y) {
      float yv[VEC];
      if (VEC == 4) { const float4 q = load4<T>(y + at + c); yv[0] = q.x; yv[1 % VEC] = q.y; yv[2 % VEC] = q.z; yv[3 % VEC] = q.w; }
      else yv[0] = to_f32<T>(y[at + c]);
#pragma unroll
      for (int e = 0; e < VEC; e++) v[e] = fmaf(a.mult, yv[e], v[e]);
    }
    if (a.add_vec) {
#pragma unroll
      for (int e = 0; e < VEC; e++) v[e] += a.add_vec[c + e];
    }
    if (a.dst && (y || a.add_vec || a.dst != a.src)) {
      if (VEC == 4) *(float4 *)(a.dst + at + c) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
      else a.dst[at + c] = v[0];
    }
    if (n_hist > 0) {       // the mix over the history; an entry that is dst is this thread's own fresh value
      float m[VEC];
#pragma unroll
      for (int e = 0; e < VEC; e++) m[e] = 0.0f;
      for (int j = 0; j < n_hist; j++) {
        const float *hj = a.hist + (int64_t)j * a.hist_stride;
        float hv[VEC];
        if (hj == a.dst) {
#pragma unroll
          for (int e = 0; e < VEC; e++) hv[e] = v[e];
        } else if (VEC == 4) {
          const float4 q = *(const float4 *)(hj + at + c);
          hv[0] = q.x; hv[1 % VEC] = q.y; hv[2 % VEC] = q.z; hv[3 % VEC] = q.w;
        } else {
          hv[0] = hj[at + c];
        }
#pragma unroll
        for (int e = 0; e < VEC; e++) m[e] = fmaf(mix[j], hv[e], m[e]);
      }
#pragma unroll
      for (int e = 0; e < VEC; e++) v[e] = m[e];
      if (a.mixed) {
        if (VEC == 4) *(float4 *)(a.mixed + at + c) = make_float4(v[0], v[1 % VEC], v[2 % VEC], v[3 % VEC]);
        else a.mixed[at + c] = v[0];
      }
    }
#pragma unroll
    for (int e = 0; e < VEC; e++) {
      row[c + e] = v[e];
      ss = fmaf(v[e], v[e], ss);
    }
  }
  if (a.next_out == nullptr) return;
  const float inv = rsqrtf_exact(block_sum(ss, red) / (float)width + a.eps);
  T *out = (T *)a.next_out;
  for (int c = threadIdx.x * VEC; c < width; c += blockDim.x * VEC) {     // every thread re-reads the columns it wrote itself
    if (VEC == 4) {
      const float4 w = *(const float4 *)(a.next_w + c);
      store4<T>(out + at + c, make_float4(row[c] * inv * w.x, row[c + 1 % VEC] * inv * w.y, row[c + 2 % VEC] * inv * w.z, row[c + 3 % VEC] * inv * w.w));
    } else {
      out[at + c] = from_f32<T>(row[c] * inv * a.next_w[c]);
    }
  }
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_embed_scaled(const void *table, int dtype, const int32_t *ids, float scale, float *out, int n_tok, int width,
                                    int64_t stream) {
  if (n_tok <= 0) return 0;
  const int th = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  SEQ_DISPATCH_DTYPE(dtype, (embed_scaled_kernel<T><<<n_tok, th, 0, (cudaStream_t)stream>>>((const T *)table, ids, scale, out, width)));
  return launch_status();
}

extern "C" int mrs_seq_embed_pair(const void *table, const void *pairs, int dtype, const int32_t *ids, float scale, int64_t buckets,
                                  int64_t mul_prev, int64_t mul_cur, int32_t *prev_state, const int32_t *cu_tok, const int32_t *past,
                                  const int32_t *slot, const int32_t *seq_of_tok, float *out, int n_tok, int width, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (!table || !pairs || !prev_state || buckets <= 0 || width <= 0) return -2;
  const int th = width >= 1024 ? 256 : (width >= 256 ? 128 : 64);
  SEQ_DISPATCH_DTYPE(dtype, (embed_pair_kernel<T><<<n_tok, th, 0, (cudaStream_t)stream>>>((const T *)table, (const T *)pairs, ids, scale, buckets,
                                                                                        mul_prev, mul_cur, prev_state, cu_tok, past, slot,
                                                                                        seq_of_tok, out, width)));
  return launch_status();
}

extern "C" int mrs_seq_rms_residual(const mrs_seq_rms_residual_args *args, int64_t stream) {
  const mrs_seq_rms_residual_args &a = *args;
  if (a.n_tok <= 0) return 0;
  if (!a.src || a.width <= 0 || (a.hist && (a.n_hist < 1 || a.n_hist > 128 || !a.mix)) || (a.next_out && !a.next_w)) return -2;
  const size_t bytes = (size_t)a.width * sizeof(float);
  if (bytes > 200 * 1024) return -2;
  auto al = [](const void *p) { return ((uintptr_t)p & 15) == 0; };
  const bool vec = a.width % 4 == 0 && al(a.src) && al(a.dst) && al(a.y) && al(a.hist) && a.hist_stride % 4 == 0 && al(a.mixed) &&
                   al(a.next_w) && al(a.next_out);      // post_w and add_vec are read one element at a time
  const int items = vec ? a.width / 4 : a.width;
  int th = 64;
  while (th < 1024 && th * (a.n_tok <= 64 ? 1 : 2) < items) th *= 2;    // short batches: one item per thread where possible
  cudaStream_t st = (cudaStream_t)stream;
#define SEQ_RES(V)                                                                                          \
  {                                                                                                         \
    auto kern = rms_residual_kernel<T, V>;                                                                  \
    static size_t allowed = 48 * 1024;                                                                      \
    if (bytes > allowed) {                                                                                  \
      const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes); \
      if (e != cudaSuccess) return (int)e;                                                                  \
      allowed = bytes;                                                                                      \
    }                                                                                                       \
    kern<<<a.n_tok, th, bytes, st>>>(a);                                                                    \
  }
  SEQ_DISPATCH_DTYPE(a.dtype, {
    if (vec) SEQ_RES(4) else SEQ_RES(1)
  });
#undef SEQ_RES
  return launch_status();
}
