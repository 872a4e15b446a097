// seq_common.cuh — helpers shared by the sequence-mixer kernels (libmrs_b200_seq.so): activation storage
// types (bf16 or f32, picked by the dtype code of the C ABI), exact f32 activations, block reductions and the
// per-step batch description.  Everything that the kernels accumulate, normalise or carry from token to token is
// f32; only tensors that a matrix product reads or writes take the activation type.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../../include/mrs_b200_seq.h"

namespace seq {

// ---- storage types ----------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- exact activations (no fast-math intrinsics: the f32 mode is held to f32 rounding) ----------------
__device__ __forceinline__ float sigmoid_f(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float gelu_erf_f(float z) { return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f)); }
__device__ __forceinline__ float relu_sq_f(float z) { return z > 0.0f ? z * z : 0.0f; }
__device__ __forceinline__ float rsqrtf_exact(float x) { return 1.0f / sqrtf(x); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float apply_act(float z, int act) {
  switch (act) {
    case MRS_SEQ_ACT_SILU: return silu_f(z);
    case MRS_SEQ_ACT_GELU_TANH: return gelu_tanh_f(z);
    case MRS_SEQ_ACT_SIGMOID: return sigmoid_f(z);
    case MRS_SEQ_ACT_GELU_ERF: return gelu_erf_f(z);
    case MRS_SEQ_ACT_RELU_SQ: return relu_sq_f(z);
    default: return z;
  }
}

// gate and up halves of a gated feed-forward joined by a rule (mrs_seq_glu_rule)
__device__ __forceinline__ float glu_join(float g, float u, const mrs_seq_glu_rule &r) {
  if (r.act == MRS_SEQ_GLU_CAPPED) {
    g = fminf(g, r.limit);
    u = fminf(fmaxf(u, -r.limit), r.limit);
    return g * sigmoid_f(r.slope * g) * (u + r.shift);
  }
  return apply_act(g, r.act) * u;
}

// ---- reductions -------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) x += __shfl_xor_sync(0xffffffffu, x, m);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int m = 16; m > 0; m >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, m));
  return x;
}
// sum over the block; `red` is 33 floats of shared memory; every thread gets the result
__device__ __forceinline__ float block_sum(float x, float *red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  x = warp_sum(x);
  __syncthreads();   // `red` may still be read from an earlier call
  if (lane == 0) red[w] = x;
  __syncthreads();
  if (w == 0) {
    float y = lane < nw ? red[lane] : 0.0f;
    y = warp_sum(y);
    if (lane == 0) red[32] = y;
  }
  __syncthreads();
  return red[32];
}

// ---- 16-byte loads: dot of 16 bytes of a row with f32 values, and two neighbouring elements ----------
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };
template <typename T> __device__ __forceinline__ float dot16(const float *q, const T *k);
template <> __device__ __forceinline__ float dot16<float>(const float *q, const float *k) {
  const float4 a = *(const float4 *)k, b = *(const float4 *)q;
  return fmaf(a.x, b.x, fmaf(a.y, b.y, fmaf(a.z, b.z, a.w * b.w)));
}
template <> __device__ __forceinline__ float dot16<__nv_bfloat16>(const float *q, const __nv_bfloat16 *k) {
  const uint4 raw = *(const uint4 *)k;
  const __nv_bfloat162 *h = (const __nv_bfloat162 *)&raw;
  const float4 b0 = *(const float4 *)q, b1 = *(const float4 *)(q + 4);
  const float2 k0 = __bfloat1622float2(h[0]), k1 = __bfloat1622float2(h[1]), k2 = __bfloat1622float2(h[2]), k3 = __bfloat1622float2(h[3]);
  return fmaf(k0.x, b0.x, fmaf(k0.y, b0.y, fmaf(k1.x, b0.z, k1.y * b0.w))) + fmaf(k2.x, b1.x, fmaf(k2.y, b1.y, fmaf(k3.x, b1.z, k3.y * b1.w)));
}
template <typename T> __device__ __forceinline__ float2 load2(const T *p);
template <> __device__ __forceinline__ float2 load2<float>(const float *p) { return *(const float2 *)p; }
template <> __device__ __forceinline__ float2 load2<__nv_bfloat16>(const __nv_bfloat16 *p) { return __bfloat1622float2(*(const __nv_bfloat162 *)p); }


// four neighbouring elements (the pointer is 4-element aligned)
template <typename T> __device__ __forceinline__ float4 load4(const T *p);
template <> __device__ __forceinline__ float4 load4<float>(const float *p) { return *(const float4 *)p; }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16 *p) {
  const uint2 raw = *(const uint2 *)p;
  const float2 a = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.x), b = __bfloat1622float2(*(const __nv_bfloat162 *)&raw.y);
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void store4(T *p, float4 v);
template <> __device__ __forceinline__ void store4<float>(float *p, float4 v) { *(float4 *)p = v; }
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16 *p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *(const uint32_t *)&a;
  raw.y = *(const uint32_t *)&b;
  *(uint2 *)p = raw;
}
__device__ __forceinline__ float4 act4(float4 v, int act) {
  return make_float4(apply_act(v.x, act), apply_act(v.y, act), apply_act(v.z, act), apply_act(v.w, act));
}

// dot of one weight row (global) with x (shared, f32) across a warp; every lane gets the sum
template <typename T>
__device__ __forceinline__ float warp_row_dot(const T *__restrict__ w, const float *__restrict__ x, int n, int lane, bool vec) {
  constexpr int N = Vec16<T>::N;
  float a = 0.0f, b = 0.0f;
  if (vec) {
    int c = lane * N;
    for (; c + 32 * N < n; c += 64 * N) {
      a += dot16<T>(x + c, w + c);
      b += dot16<T>(x + c + 32 * N, w + c + 32 * N);
    }
    if (c < n) a += dot16<T>(x + c, w + c);
  } else {
    for (int c = lane; c < n; c += 32) a = fmaf(to_f32<T>(w[c]), x[c], a);
  }
  return warp_sum(a + b);
}

// launch helper: a C-ABI function returns the CUDA error of its launches as an int (0 = ok)
inline int launch_status() { return (int)cudaGetLastError(); }

}  // namespace seq

#define SEQ_DISPATCH_DTYPE(dtype, ...)                                    \
  do {                                                                    \
    if ((dtype) == MRS_SEQ_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else if ((dtype) == MRS_SEQ_F32) { using T = float; __VA_ARGS__; }     \
    else return -1;                                                       \
  } while (0)
