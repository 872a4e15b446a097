// scan.cu — gated linear recurrences with an f32 state per (sequence, head), and what surrounds them: the short
// causal convolution with its carried inputs, the step-size / decay preparation of a selective state space, the
// gated group RMS norm of the recurrence's output, and the split GLU.
//
//   S_t = a_t S_(t-1) + b_t k_t v_t^T ,  o_t = S_t^T q_t + skip v_t
//
// covers linear attention with a fixed per-head decay (a_t constant, b_t = 1, silu on q / k / v), the state-space
// form (k = B, q = C, v = x, a_t = exp(-exp(A_log) dt_t), b_t = dt_t, skip = D) and — template flag VD — a forget gate
// per state ROW, either with keys of their own (gated linear attention: S_t = diag(f_t) S_(t-1) + k_t v_t^T) or one that
// also decides what is written (k == NULL: S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, the key is the gate's complement and
// is formed here, in f32, from the same staged row).  Queries can carry a constant factor (q_scale).  The same kernel runs a prompt
// portion and a single decoded token: the state is read from the sequence's slot (or taken as zero when the
// sequence starts), advanced token by token in registers, and written back.
#include "seq_common.cuh"

namespace seq {

// One CTA: one sequence, one head, CW state columns.  Thread (col, part) keeps rows [part * RK, part * RK + RK) of its
// column in registers; the `parts` partitions of a column sit in neighbouring lanes, so the dot with q ends in a few
// shuffles.  Tokens go through in rounds of TC: while one round runs out of f32 shared memory, the next round's
// q / k / v / a / b stream into a raw staging area (cp.async, 16 bytes at a time when the rows are aligned), and are
// converted (and activated) between rounds — the global latency hides behind the token loop.
// two f32 lanes per instruction (sm_100 packed arithmetic): the scan's state update and dot are FMA-issue-bound
__device__ __forceinline__ uint64_t pack2(float x, float y) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float &x, float &y) { asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v)); }
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

__device__ __forceinline__ void cp_async16(void *dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void *dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <typename T, int RK, int TC, bool VD>
__global__ void __launch_bounds__(256, RK <= 16 ? (VD ? 2 : 3) : 1) linear_scan_kernel(const mrs_seq_scan_args a, int parts, int cw, int aligned, int mode) {
  // mode 0: the whole portion of a sequence, state from / to its slot.  Long portions are cut into segments of
  // a.seg_len tokens that run side by side: mode 1 advances a ZERO state over one segment and leaves it, with the
  // segment's product of decays, in a.seg_state / a.seg_decay; a small kernel then chains the segments (and the slot's
  // state) into every segment's true start state; mode 2 runs the segment again from that start and writes the outputs.
  extern __shared__ __align__(16) float smem[];
  constexpr int N = 16 / (int)sizeof(T);     // elements per 16 bytes
  const int b = mode ? blockIdx.z / a.n_segs : blockIdx.z, seg = mode ? blockIdx.z % a.n_segs : 0;
  const int h = blockIdx.y, col0 = blockIdx.x * cw;
  int t0 = a.cu_tok[b], t1 = a.cu_tok[b + 1];
  if (mode) {
    t0 += seg * a.seg_len;
    t1 = min(t1, t0 + a.seg_len);
  }
  if (t1 <= t0) return;
  const int dk = a.dk, dv = a.dv, heads = a.heads, nth = blockDim.x;
  const int g = h / (heads / a.qk_groups);
  const int part = threadIdx.x % parts, cl = threadIdx.x / parts;
  constexpr int PS = RK + 4;             // padded partition stride (floats): 16-byte aligned, conflict-free
  const int dks = parts * PS;
  const int dkr = (dk + N - 1) / N * N, cwr = (cw + N - 1) / N * N;      // raw row lengths (elements), 16-byte multiples
  float *qs = smem, *ks = qs + TC * dks, *vs = ks + TC * dks, *os = vs + TC * cw, *as = os + TC * cw, *bs = as + TC;
  float *ra = bs + TC, *rb = ra + TC;
  float *ds = rb + TC, *rd = ds + (VD ? TC * dks : 0);      // per-row decays: working set (laid out like ks) and raw staging
  T *rq = (T *)(rd + (VD ? TC * dkr : 0)), *rk = rq + TC * dkr, *rv = rk + TC * dkr;
  float *state = mode ? a.seg_state + ((int64_t)blockIdx.z * heads + h) * dk * dv : a.state + ((int64_t)a.slot[b] * heads + h) * dk * dv;
  float decay_product = 1.0f;
  uint64_t dp2[VD ? RK / 2 : 1];      // per-row products of the decays over a segment (mode 1 with per-row decays)
#pragma unroll
  for (int r = 0; r < (VD ? RK / 2 : 1); r++) dp2[r] = pack2(1.0f, 1.0f);

  uint64_t S[RK / 2];      // the state column's rows as packed pairs (row 2i, row 2i + 1)
  if (mode == 2 || (mode == 0 && a.past[b] > 0)) {   // stage the tile [dk, cw] through shared memory so the global reads run along columns
    float *tile = smem;
    if (dv % 4 == 0 && cw % 4 == 0 && ((uintptr_t)state & 15) == 0) {   // all 16-byte pieces in flight at once
      const int per = cw / 4;
      for (int e = threadIdx.x; e < parts * RK * per; e += nth) {
        const int r = e / per, c = (e % per) * 4;
        if (r < dk && col0 + c < dv) cp_async16(tile + r * cw + c, state + (int64_t)r * dv + col0 + c);
        else *(float4 *)(tile + r * cw + c) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
      cp_async_commit();
      cp_async_wait_all();
    } else {
      for (int e = threadIdx.x; e < parts * RK * cw; e += nth) {
        const int r = e / cw, c = e % cw;
        tile[e] = (r < dk && col0 + c < dv) ? state[(int64_t)r * dv + col0 + c] : 0.0f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < RK; r += 2) S[r / 2] = pack2(tile[(part * RK + r) * cw + cl], tile[(part * RK + r + 1) * cw + cl]);
    __syncthreads();
  } else {
#pragma unroll
    for (int r = 0; r < RK / 2; r++) S[r] = 0ull;
  }
  for (int e = threadIdx.x; e < 2 * TC * dks; e += nth) qs[e] = 0.0f;     // rows past dk stay zero for good
  if (VD)
    for (int e = threadIdx.x; e < TC * dks; e += nth) ds[e] = 0.0f;
  const float skip = a.skip ? a.skip[h] : 0.0f;
  const bool own_k = !VD || a.k != nullptr;      // per-row decays with keys of their own, or keys that are the decays' complement
  const float q_scale = a.q_scale != 0.0f ? a.q_scale : 1.0f;
  const T *q = (const T *)a.q + g * dk, *k = own_k ? (const T *)a.k + g * dk : nullptr, *v = (const T *)a.v + h * dv + col0;
  const float *dvec = VD ? a.decay_vec + (int64_t)h * dk : nullptr;
  const bool dvec_aligned = VD && dk % 4 == 0 && ((uintptr_t)a.decay_vec & 15) == 0;
  const int vcols = min(cw, dv - col0);

  auto issue = [&](int c0) {      // round starting at token c0 -> raw staging
    const int n = min(TC, t1 - c0);
    if (aligned) {
      const int per = dkr / N;
      for (int e = threadIdx.x; e < n * per; e += nth) {
        const int i = e / per, j = e % per;
        cp_async16(rq + i * dkr + j * N, q + (int64_t)(c0 + i) * a.q_ld + j * N);
        if (own_k) cp_async16(rk + i * dkr + j * N, k + (int64_t)(c0 + i) * a.k_ld + j * N);
      }
      const int perv = vcols / N;
      for (int e = threadIdx.x; e < n * perv; e += nth) {
        const int i = e / perv, j = e % perv;
        cp_async16(rv + i * cwr + j * N, v + (int64_t)(c0 + i) * a.v_ld + j * N);
      }
    } else {
      for (int e = threadIdx.x; e < n * dk; e += nth) {
        const int i = e / dk, d = e % dk;
        rq[i * dkr + d] = q[(int64_t)(c0 + i) * a.q_ld + d];
        if (own_k) rk[i * dkr + d] = k[(int64_t)(c0 + i) * a.k_ld + d];
      }
      for (int e = threadIdx.x; e < n * vcols; e += nth) {
        const int i = e / vcols, c = e % vcols;
        rv[i * cwr + c] = v[(int64_t)(c0 + i) * a.v_ld + c];
      }
    }
    if (VD) {
      if (dvec_aligned) {
        const int per = dk / 4;
        for (int e = threadIdx.x; e < n * per; e += nth) {
          const int i = e / per, j = e % per;
          cp_async16(rd + i * dkr + j * 4, dvec + (int64_t)(c0 + i) * heads * dk + j * 4);
        }
      } else {
        for (int e = threadIdx.x; e < n * dk; e += nth) {
          const int i = e / dk, d = e % dk;
          rd[i * dkr + d] = dvec[(int64_t)(c0 + i) * heads * dk + d];
        }
      }
    }
    if (threadIdx.x < n) {
      const int64_t th = (int64_t)(c0 + threadIdx.x) * heads + h;
      if (a.decay_tok) cp_async4(ra + threadIdx.x, a.decay_tok + th);
      if (a.scale_tok) cp_async4(rb + threadIdx.x, a.scale_tok + th);
    }
    cp_async_commit();
  };

  issue(t0);
  for (int c0 = t0; c0 < t1; c0 += TC) {
    const int n = min(TC, t1 - c0);
    cp_async_wait_all();
    __syncthreads();
    {   // raw -> f32 working set (activation applied here)
      const int per = dkr / N;
      for (int e = threadIdx.x; e < n * per; e += nth) {
        const int i = e / per, d0 = (e % per) * N;
        const int at = i * dks + (d0 / RK) * PS + d0 % RK;
#pragma unroll
        for (int x = 0; x < N; x++) {
          const bool in = d0 + x < dk;
          qs[at + x] = in ? apply_act(to_f32<T>(rq[i * dkr + d0 + x]), a.act) * q_scale : 0.0f;
          if (VD) {
            const float f = in ? rd[i * dkr + d0 + x] : 0.0f;
            ds[at + x] = f;
            ks[at + x] = !in ? 0.0f : (own_k ? apply_act(to_f32<T>(rk[i * dkr + d0 + x]), a.act) : 1.0f - f);
          } else {
            ks[at + x] = in ? apply_act(to_f32<T>(rk[i * dkr + d0 + x]), a.act) : 0.0f;
          }
        }
      }
      for (int e = threadIdx.x; e < n * cw; e += nth) {
        const int i = e / cw, c = e % cw;
        vs[e] = c < vcols ? apply_act(to_f32<T>(rv[i * cwr + c]), a.act) : 0.0f;
      }
      if (threadIdx.x < n) {
        as[threadIdx.x] = VD ? 1.0f : (a.decay_tok ? ra[threadIdx.x] : a.decay_head[h]);
        bs[threadIdx.x] = a.scale_tok ? rb[threadIdx.x] : 1.0f;
      }
    }
    __syncthreads();
    if (c0 + TC < t1) issue(c0 + TC);
    // four tokens per pass: the state's chain through them is short (two dependent operations per token and row), while
    // their shared-memory reads, dot products and shuffle trees are independent and overlap
    for (int i0 = 0; i0 < n; i0 += 4) {
      float vv[4];
      uint64_t av2[4], bv2[4], acc2[4];
      bool lv[4];
#pragma unroll
      for (int u = 0; u < 4; u++) {
        const bool live = i0 + u < n;
        lv[u] = live;          // a missing token leaves the state alone (rows past n hold old, finite data)
        vv[u] = vs[(i0 + u) * cw + cl];
        const float av = live ? as[i0 + u] : 1.0f, bv = live ? bs[i0 + u] * vv[u] : 0.0f;
        av2[u] = pack2(av, av);
        bv2[u] = pack2(bv, bv);
        acc2[u] = 0ull;
        decay_product *= av;
      }
#pragma unroll
      for (int r = 0; r < RK; r += 4) {
        ulonglong2 k4[4], q4[4];               // four rows of k / q as two packed pairs
#pragma unroll
        for (int u = 0; u < 4; u++) {
          k4[u] = *(const ulonglong2 *)(ks + (i0 + u) * dks + part * PS + r);
          if (mode != 1) q4[u] = *(const ulonglong2 *)(qs + (i0 + u) * dks + part * PS + r);
        }
        uint64_t s01 = S[r / 2], s23 = S[r / 2 + 1];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          if (VD) {      // this row's own decay; a missing token keeps the state as it is
            const ulonglong2 d4 = *(const ulonglong2 *)(ds + (i0 + u) * dks + part * PS + r);
            const uint64_t d01 = lv[u] ? d4.x : av2[u], d23 = lv[u] ? d4.y : av2[u];
            s01 = fma2(k4[u].x, bv2[u], mul2(d01, s01));
            s23 = fma2(k4[u].y, bv2[u], mul2(d23, s23));
            if (mode == 1) {
              dp2[VD ? r / 2 : 0] = mul2(dp2[VD ? r / 2 : 0], d01);
              dp2[VD ? r / 2 + 1 : 0] = mul2(dp2[VD ? r / 2 + 1 : 0], d23);
            }
          } else {
            s01 = fma2(k4[u].x, bv2[u], mul2(av2[u], s01));
            s23 = fma2(k4[u].y, bv2[u], mul2(av2[u], s23));
          }
          if (mode != 1) acc2[u] = fma2(s01, q4[u].x, fma2(s23, q4[u].y, acc2[u]));
        }
        S[r / 2] = s01;
        S[r / 2 + 1] = s23;
      }
      if (mode != 1) {
        float acc[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          float lo, hi;
          unpack2(acc2[u], lo, hi);
          acc[u] = lo + hi;
        }
        for (int m = 1; m < parts; m <<= 1) {
#pragma unroll
          for (int u = 0; u < 4; u++) acc[u] += __shfl_xor_sync(0xffffffffu, acc[u], m);
        }
        if (part == 0) {
#pragma unroll
          for (int u = 0; u < 4; u++)
            if (i0 + u < n) os[(i0 + u) * cw + cl] = fmaf(skip, vv[u], acc[u]);
        }
      }
    }
    __syncthreads();
    if (mode != 1)
      for (int e = threadIdx.x; e < n * cw; e += nth) {
        const int i = e / cw, c = e % cw;
        if (c < vcols) a.out[(int64_t)(c0 + i) * heads * dv + h * dv + col0 + c] = os[e];
      }
  }
  __syncthreads();
  if (VD) {
    if (mode == 1 && blockIdx.x == 0 && cl == 0) {      // seg_decay holds one product per state row
      float *out = a.seg_decay + ((int64_t)blockIdx.z * heads + h) * dk;
#pragma unroll
      for (int r = 0; r < RK; r += 2) {
        float lo, hi;
        unpack2(dp2[VD ? r / 2 : 0], lo, hi);
        if (part * RK + r < dk) out[part * RK + r] = lo;
        if (part * RK + r + 1 < dk) out[part * RK + r + 1] = hi;
      }
    }
  } else if (mode == 1 && blockIdx.x == 0 && threadIdx.x == 0) a.seg_decay[(int64_t)blockIdx.z * heads + h] = decay_product;
  if (mode != 2) {   // the state goes back the way it came
    float *tile = smem;
#pragma unroll
    for (int r = 0; r < RK; r += 2) {
      float lo, hi;
      unpack2(S[r / 2], lo, hi);
      tile[(part * RK + r) * cw + cl] = lo;
      tile[(part * RK + r + 1) * cw + cl] = hi;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < parts * RK * cw; e += nth) {
      const int r = e / cw, c = e % cw;
      if (r < dk && col0 + c < dv) state[(int64_t)r * dv + col0 + c] = tile[e];
    }
  }
}

// chains the segments of every sequence: seg_state[seg] <- the state before segment seg; the slot gets the final state
__global__ void scan_chain_kernel(const mrs_seq_scan_args a) {
  const int b = blockIdx.z, h = blockIdx.y, e = blockIdx.x * blockDim.x + threadIdx.x, per = a.dk * a.dv;
  if (e >= per) return;
  const int len = a.cu_tok[b + 1] - a.cu_tok[b];
  if (len <= 0) return;
  const int nseg = (len + a.seg_len - 1) / a.seg_len;
  float *slot_state = a.state + ((int64_t)a.slot[b] * a.heads + h) * per + e;
  float run = a.past[b] > 0 ? *slot_state : 0.0f;
  for (int s = 0; s < nseg; s++) {
    const int64_t z = (int64_t)b * a.n_segs + s;
    float *p = a.seg_state + (z * a.heads + h) * per + e;
    const float local = *p;
    *p = run;
    run = fmaf(a.decay_vec ? a.seg_decay[(z * a.heads + h) * a.dk + e / a.dv] : a.seg_decay[z * a.heads + h], run, local);
  }
  *slot_state = run;
}

template <typename T, int RK, int TC, bool VD>
static int launch_scan(const mrs_seq_scan_args &a, cudaStream_t st) {
  constexpr int N = 16 / (int)sizeof(T);
  int parts = 1;
  while (parts * RK < a.dk) parts <<= 1;
  if (parts > 32) return -2;
  const int unit = 32 / parts > N ? 32 / parts : N;               // columns per CTA: whole warps, whole 16-byte groups
  int cw = min(256 / parts, (a.dv + unit - 1) / unit * unit);
  if (cw < unit) cw = unit;
  while (cw / 2 >= unit && (cw / 2) % unit == 0 && (cw / 2) * parts >= 64 && (int64_t)((a.dv + cw - 1) / cw) * a.heads * a.n_seq * (a.n_segs > 1 ? a.n_segs : 1) < 148) cw /= 2;   // fill the SMs
  if (cw * parts > 256 || (cw * parts) % 32) return -2;
  const int dks = parts * (RK + 4), dkr = (a.dk + N - 1) / N * N, cwr = (cw + N - 1) / N * N;
  const size_t work = (size_t)(2 * TC * dks + 2 * TC * cw + 4 * TC + (VD ? TC * dks + TC * dkr : 0)) * sizeof(float) +
                      (size_t)(2 * TC * dkr + TC * cwr) * sizeof(T);
  const size_t tile = (size_t)parts * RK * cw * sizeof(float);
  const size_t bytes = work > tile ? work : tile;
  const bool aligned = a.dk % N == 0 && a.dv % N == 0 && cw % N == 0 && a.q_ld % N == 0 && (!a.k || a.k_ld % N == 0) && a.v_ld % N == 0 &&
                       (uintptr_t)a.q % 16 == 0 && (uintptr_t)a.k % 16 == 0 && (uintptr_t)a.v % 16 == 0;
  auto kern = linear_scan_kernel<T, RK, TC, VD>;
  static size_t allowed = 48 * 1024;      // per instantiation; raised once per size, so a captured step repeats no attribute call
  if (bytes > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
    allowed = bytes;
  }
  if (a.n_segs > 1 && a.seg_state && a.seg_decay && a.seg_len > 0) {
    dim3 grid((a.dv + cw - 1) / cw, a.heads, a.n_seq * a.n_segs);
    kern<<<grid, cw * parts, bytes, st>>>(a, parts, cw, aligned ? 1 : 0, 1);
    const int per = a.dk * a.dv;
    scan_chain_kernel<<<dim3((per + 255) / 256, a.heads, a.n_seq), 256, 0, st>>>(a);
    kern<<<grid, cw * parts, bytes, st>>>(a, parts, cw, aligned ? 1 : 0, 2);
    return launch_status();
  }
  dim3 grid((a.dv + cw - 1) / cw, a.heads, a.n_seq);
  kern<<<grid, cw * parts, bytes, st>>>(a, parts, cw, aligned ? 1 : 0, 0);
  return launch_status();
}

// ---- short causal convolution ------------------------------------------------------------------------------------
// one thread per (token, channel): taps reach back into the portion or, before its start, into the carried inputs
template <typename T>
__global__ void causal_conv_kernel(const T *__restrict__ in, int64_t in_ld, int col0, const float *__restrict__ taps,
                                   const float *__restrict__ bias, int channels, int n_taps, int act,
                                   const float *__restrict__ conv_state, const int32_t *__restrict__ cu_tok,
                                   const int32_t *__restrict__ past, const int32_t *__restrict__ slot,
                                   const int32_t *__restrict__ seq_of_tok, T *__restrict__ out) {
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int s = seq_of_tok[t], first = cu_tok[s], i = t - first, carried = n_taps - 1;
  const bool has_past = past[s] > 0;
  const float *st = conv_state + (int64_t)slot[s] * carried * channels;
  float acc = bias ? bias[c] : 0.0f;
  for (int j = 0; j < n_taps; j++) {
    const int src = i - carried + j;   // index inside the portion
    float x;
    if (src >= 0) x = to_f32<T>(in[(int64_t)(first + src) * in_ld + col0 + c]);
    else x = has_past ? st[(int64_t)(carried + src) * channels + c] : 0.0f;
    acc = fmaf(taps[(int64_t)c * n_taps + j], x, acc);
  }
  out[(int64_t)t * channels + c] = from_f32<T>(apply_act(acc, act));
}

// Four neighbouring channels per thread (16-byte accesses) and CONV_TB neighbouring tokens per CTA, when rows and channel
// counts are 4-element aligned and there are at most 8 taps: the thread walks its tokens with the last n_taps - 1 inputs in
// registers, so every input is loaded once (not once per tap) and the index chain token -> sequence -> first row / slot is
// followed once per CTA (and again where a new sequence starts inside the block), not once per output.
constexpr int CONV_TB = 16, CONV_MAXC = 7;
template <typename T>
__global__ void __launch_bounds__(128) causal_conv_vec_kernel(const T *__restrict__ in, int64_t in_ld, int col0, const float *__restrict__ taps,
                                       const float *__restrict__ bias, int channels, int n_taps, int act,
                                       const float *__restrict__ conv_state, const int32_t *__restrict__ cu_tok,
                                       const int32_t *__restrict__ past, const int32_t *__restrict__ slot,
                                       const int32_t *__restrict__ seq_of_tok, int n_tok, T *__restrict__ out) {
  const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
  if (c >= channels) return;
  const int t0 = blockIdx.x * CONV_TB, t1 = min(n_tok, t0 + CONV_TB), carried = n_taps - 1, lead = CONV_MAXC - carried;
  float w[4][CONV_MAXC + 1];       // taps right-aligned: w[.][lead + j] = tap j
#pragma unroll
  for (int k = 0; k <= CONV_MAXC; k++)
#pragma unroll
    for (int e = 0; e < 4; e++) w[e][k] = k >= lead ? taps[(int64_t)(c + e) * n_taps + k - lead] : 0.0f;
  const float4 b4 = bias ? *(const float4 *)(bias + c) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
  float4 hist[CONV_MAXC];          // hist[CONV_MAXC - 1] = the input before the current token
  int s = -1;
  for (int t = t0; t < t1; t++) {
    const int st = seq_of_tok[t];
    if (st != s) {                 // the block's first token, or a sequence starts here: fetch the inputs before it
      s = st;
      const int first = cu_tok[s], i = t - first;
      const bool has_past = past[s] > 0;
      const float *cs = conv_state + (int64_t)slot[s] * carried * channels;
#pragma unroll
      for (int k = 0; k < CONV_MAXC; k++) {
        const int src = i - CONV_MAXC + k;            // k >= lead: the carried range
        if (k < lead) hist[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        else if (src >= 0) hist[k] = load4<T>(in + (int64_t)(first + src) * in_ld + col0 + c);
        else if (has_past) hist[k] = *(const float4 *)(cs + (int64_t)(carried + src) * channels + c);
        else hist[k] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    }
    const float4 x = load4<T>(in + (int64_t)t * in_ld + col0 + c);
    float4 acc = b4;
#pragma unroll
    for (int k = 0; k < CONV_MAXC; k++) {
      acc.x = fmaf(w[0][k], hist[k].x, acc.x);
      acc.y = fmaf(w[1][k], hist[k].y, acc.y);
      acc.z = fmaf(w[2][k], hist[k].z, acc.z);
      acc.w = fmaf(w[3][k], hist[k].w, acc.w);
    }
    acc.x = fmaf(w[0][CONV_MAXC], x.x, acc.x);
    acc.y = fmaf(w[1][CONV_MAXC], x.y, acc.y);
    acc.z = fmaf(w[2][CONV_MAXC], x.z, acc.z);
    acc.w = fmaf(w[3][CONV_MAXC], x.w, acc.w);
    store4<T>(out + (int64_t)t * channels + c, act4(acc, act));
#pragma unroll
    for (int k = 0; k + 1 < CONV_MAXC; k++) hist[k] = hist[k + 1];
    hist[CONV_MAXC - 1] = x;
  }
}

// runs after the convolution: the carried inputs become the last n_taps-1 inputs of the sequence
template <typename T>
__global__ void conv_state_advance_kernel(const T *__restrict__ in, int64_t in_ld, int col0, int channels, int n_taps,
                                          float *__restrict__ conv_state, const int32_t *__restrict__ cu_tok,
                                          const int32_t *__restrict__ past, const int32_t *__restrict__ slot) {
  const int s = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int first = cu_tok[s], n = cu_tok[s + 1] - first, carried = n_taps - 1;
  if (n <= 0) return;
  const bool has_past = past[s] > 0;
  float *st = conv_state + (int64_t)slot[s] * carried * channels;
  for (int j = 0; j < carried; j++) {   // ascending: entry j reads old entry j + n, never one already rewritten
    const int src = n - carried + j;
    float x;
    if (src >= 0) x = to_f32<T>(in[(int64_t)(first + src) * in_ld + col0 + c]);
    else x = has_past ? st[(int64_t)(carried + src) * channels + c] : 0.0f;
    st[(int64_t)j * channels + c] = x;
  }
}

template <typename T>
__global__ void ssm_steps_kernel(const T *__restrict__ in, int64_t in_ld, int col0, const float *__restrict__ bias,
                                 const float *__restrict__ a_log, int heads, int n_tok, float *__restrict__ step,
                                 float *__restrict__ decay) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_tok * heads) return;
  const int t = e / heads, h = e % heads;
  const float dt = softplus_f(to_f32<T>(in[(int64_t)t * in_ld + col0 + h]) + bias[h]);
  step[e] = dt;
  decay[e] = expf(-expf(a_log[h]) * dt);
}

// ---- gated group RMS norm ------------------------------------------------------------------------------------------
// one CTA per (token, group); VEC = 4: four columns per thread and pass, the row kept in registers between the passes
// when it fits (KEEP vector items per thread), so a short batch pays one round of global latency, not sixteen
template <typename T, int VEC, int KEEP>
__global__ void __launch_bounds__(1024) gated_group_norm_kernel(const float *__restrict__ x, const T *__restrict__ gate, int64_t gate_ld,
                                        const float *__restrict__ weight, T *__restrict__ out, int64_t out_ld, float out_scale, int cols,
                                        int groups, float eps, int gate_act, int gate_first) {
  __shared__ float red[33];
  const int t = blockIdx.x, gr = blockIdx.y, n = cols / groups, c0 = gr * n;
  const float *xr = x + (int64_t)t * cols + c0;
  const T *gp = gate ? gate + (int64_t)t * gate_ld + c0 : nullptr;
  T *dst = out + (int64_t)t * out_ld + c0;
  const float *w = weight + c0;
  float ss = 0.0f;
  if (VEC == 4) {
    float4 xv[KEEP], gv[KEEP];
#pragma unroll
    for (int it = 0; it < KEEP; it++) {
      const int c = (it * blockDim.x + threadIdx.x) * 4;
      if (c < n) {
        xv[it] = *(const float4 *)(xr + c);
        gv[it] = gp ? act4(load4<T>(gp + c), gate_act) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        if (gate_first) xv[it] = make_float4(xv[it].x * gv[it].x, xv[it].y * gv[it].y, xv[it].z * gv[it].z, xv[it].w * gv[it].w);
        ss += xv[it].x * xv[it].x + xv[it].y * xv[it].y + xv[it].z * xv[it].z + xv[it].w * xv[it].w;
      }
    }
    const float inv = rsqrtf_exact(block_sum(ss, red) / (float)n + eps);
#pragma unroll
    for (int it = 0; it < KEEP; it++) {
      const int c = (it * blockDim.x + threadIdx.x) * 4;
      if (c < n) {
        const float4 ww = *(const float4 *)(w + c);
        float4 r = make_float4(xv[it].x * inv * ww.x, xv[it].y * inv * ww.y, xv[it].z * inv * ww.z, xv[it].w * inv * ww.w);
        if (!gate_first) r = make_float4(r.x * gv[it].x, r.y * gv[it].y, r.z * gv[it].z, r.w * gv[it].w);
        store4<T>(dst + c, make_float4(r.x * out_scale, r.y * out_scale, r.z * out_scale, r.w * out_scale));
      }
    }
  } else {
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      float v = xr[c];
      if (gp && gate_first) v *= apply_act(to_f32<T>(gp[c]), gate_act);
      ss = fmaf(v, v, ss);
    }
    const float inv = rsqrtf_exact(block_sum(ss, red) / (float)n + eps);
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      float v = xr[c];
      const float gv = gp ? apply_act(to_f32<T>(gp[c]), gate_act) : 1.0f;
      if (gate_first) v = v * gv * inv * w[c];
      else v = v * inv * w[c] * gv;
      dst[c] = from_f32<T>(v * out_scale);
    }
  }
}

// narrow groups (a head's value size): one warp per (token, group), the group's row in registers, eight groups per CTA
template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm_warp_kernel(const float *__restrict__ x, const T *__restrict__ gate, int64_t gate_ld,
                                                                    const float *__restrict__ weight, T *__restrict__ out, int64_t out_ld,
                                                                    float out_scale, int cols, int groups, float eps, int gate_act, int gate_first,
                                                                    int64_t n_jobs) {
  constexpr int KEEP = 8;
  const int lane = threadIdx.x & 31;
  const int64_t job = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (job >= n_jobs) return;
  const int64_t t = job / groups;
  const int gr = (int)(job % groups), n = cols / groups, c0 = gr * n;
  const float *xr = x + t * cols + c0;
  const T *gp = gate ? gate + t * gate_ld + c0 : nullptr;
  T *dst = out + t * out_ld + c0;
  const float *w = weight + c0;
  float4 xv[KEEP], gv[KEEP];
  float ss = 0.0f;
#pragma unroll
  for (int it = 0; it < KEEP; it++) {
    const int c = (it * 32 + lane) * 4;
    if (c < n) {
      xv[it] = *(const float4 *)(xr + c);
      gv[it] = gp ? act4(load4<T>(gp + c), gate_act) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
      if (gate_first) xv[it] = make_float4(xv[it].x * gv[it].x, xv[it].y * gv[it].y, xv[it].z * gv[it].z, xv[it].w * gv[it].w);
      ss += xv[it].x * xv[it].x + xv[it].y * xv[it].y + xv[it].z * xv[it].z + xv[it].w * xv[it].w;
    }
  }
  const float inv = rsqrtf_exact(warp_sum(ss) / (float)n + eps);
#pragma unroll
  for (int it = 0; it < KEEP; it++) {
    const int c = (it * 32 + lane) * 4;
    if (c < n) {
      const float4 ww = *(const float4 *)(w + c);
      float4 r = make_float4(xv[it].x * inv * ww.x, xv[it].y * inv * ww.y, xv[it].z * inv * ww.z, xv[it].w * inv * ww.w);
      if (!gate_first) r = make_float4(r.x * gv[it].x, r.y * gv[it].y, r.z * gv[it].z, r.w * gv[it].w);
      store4<T>(dst + c, make_float4(r.x * out_scale, r.y * out_scale, r.z * out_scale, r.w * out_scale));
    }
  }
}

template <typename T>
__global__ void activate_cols_kernel(T *__restrict__ x, int64_t ld, int cols, int act, int vec) {
  T *row = x + (int64_t)blockIdx.x * ld;
  if (vec) {
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < cols; c += gridDim.y * blockDim.x * 4)
      store4<T>(row + c, act4(load4<T>(row + c), act));
  } else {
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < cols; c += gridDim.y * blockDim.x)
      row[c] = from_f32<T>(apply_act(to_f32<T>(row[c]), act));
  }
}

template <typename T>
__global__ void glu_split_kernel(const T *__restrict__ x, T *__restrict__ out, int half, const mrs_seq_glu_rule rule, int vec) {
  const T *row = x + (int64_t)blockIdx.x * 2 * half;
  T *dst = out + (int64_t)blockIdx.x * half;
  if (vec) {
    for (int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4; c < half; c += gridDim.y * blockDim.x * 4) {
      const float4 g = load4<T>(row + c), u = load4<T>(row + half + c);
      store4<T>(dst + c, make_float4(glu_join(g.x, u.x, rule), glu_join(g.y, u.y, rule), glu_join(g.z, u.z, rule), glu_join(g.w, u.w, rule)));
    }
  } else {
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < half; c += gridDim.y * blockDim.x)
      dst[c] = from_f32<T>(glu_join(to_f32<T>(row[c]), to_f32<T>(row[half + c]), rule));
  }
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_linear_scan(const mrs_seq_scan_args *args, int64_t stream) {
  const mrs_seq_scan_args &a = *args;
  if (a.n_tok <= 0 || a.n_seq <= 0) return 0;
  if (a.heads <= 0 || a.qk_groups <= 0 || a.heads % a.qk_groups || a.dk <= 0 || a.dv <= 0) return -2;
  if (!a.decay_tok && !a.decay_head && !a.decay_vec) return -2;
  if (a.decay_vec ? (a.decay_tok || a.decay_head || a.qk_groups != a.heads) : !a.k) return -2;      // with decay_vec, k is optional
  cudaStream_t st = (cudaStream_t)stream;
  if (a.decay_vec) {
    if (a.dk <= 128) SEQ_DISPATCH_DTYPE(a.dtype, return (launch_scan<T, 16, 16, true>(a, st)));
    if (a.dk <= 512) SEQ_DISPATCH_DTYPE(a.dtype, return (launch_scan<T, 32, 8, true>(a, st)));
    if (a.dk <= 2048) SEQ_DISPATCH_DTYPE(a.dtype, return (launch_scan<T, 64, 4, true>(a, st)));
    return -2;
  }
  if (a.dk <= 128) SEQ_DISPATCH_DTYPE(a.dtype, return (launch_scan<T, 16, 16, false>(a, st)));
  if (a.dk <= 512) SEQ_DISPATCH_DTYPE(a.dtype, return (launch_scan<T, 32, 8, false>(a, st)));
  if (a.dk <= 2048) SEQ_DISPATCH_DTYPE(a.dtype, return (launch_scan<T, 64, 4, false>(a, st)));
  return -2;
}

extern "C" int mrs_seq_causal_conv(const void *in, int64_t in_ld, int col0, int dtype, const float *taps, const float *bias,
                                   int channels, int n_taps, int act, float *conv_state, const int32_t *cu_tok,
                                   const int32_t *past, const int32_t *slot, const int32_t *seq_of_tok, int n_seq, int n_tok,
                                   void *out, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (n_taps < 1 || channels < 1) return -2;
  cudaStream_t st = (cudaStream_t)stream;
  const int th = 128;
  const bool vec = channels % 4 == 0 && in_ld % 4 == 0 && col0 % 4 == 0 && (uintptr_t)in % 16 == 0 && (uintptr_t)out % 16 == 0 &&
                   (uintptr_t)conv_state % 16 == 0 && (uintptr_t)bias % 16 == 0 && n_taps <= CONV_MAXC + 1;
  SEQ_DISPATCH_DTYPE(dtype, {
    if (vec)
      causal_conv_vec_kernel<T><<<dim3((n_tok + CONV_TB - 1) / CONV_TB, (channels / 4 + th - 1) / th), th, 0, st>>>(
          (const T *)in, in_ld, col0, taps, bias, channels, n_taps, act, conv_state, cu_tok, past, slot, seq_of_tok, n_tok, (T *)out);
    else
      causal_conv_kernel<T><<<dim3(n_tok, (channels + th - 1) / th), th, 0, st>>>((const T *)in, in_ld, col0, taps, bias, channels,
                                                                                 n_taps, act, conv_state, cu_tok, past, slot,
                                                                                 seq_of_tok, (T *)out);
    if (n_taps > 1)
      conv_state_advance_kernel<T><<<dim3((channels + th - 1) / th, n_seq), th, 0, st>>>((const T *)in, in_ld, col0, channels,
                                                                                        n_taps, conv_state, cu_tok, past, slot);
  });
  return launch_status();
}

extern "C" int mrs_seq_ssm_steps(const void *in, int64_t in_ld, int col0, int dtype, const float *bias, const float *a_log, int heads,
                                 int n_tok, float *step, float *decay, int64_t stream) {
  if (n_tok <= 0) return 0;
  const int total = n_tok * heads;
  SEQ_DISPATCH_DTYPE(dtype, (ssm_steps_kernel<T><<<(total + 127) / 128, 128, 0, (cudaStream_t)stream>>>(
                                (const T *)in, in_ld, col0, bias, a_log, heads, n_tok, step, decay)));
  return launch_status();
}

extern "C" int mrs_seq_gated_group_norm(const float *x, const void *gate, int64_t gate_ld, const float *weight, void *out, int64_t out_ld,
                                        float out_scale, int dtype, int n_tok, int cols, int groups, float eps, int gate_act,
                                        int gate_first, int64_t stream) {
  if (n_tok <= 0) return 0;
  if (groups < 1 || cols % groups) return -2;
  const int n = cols / groups;
  const bool vec = n % 4 == 0 && gate_ld % 4 == 0 && out_ld % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)gate % 16 == 0 &&
                   (uintptr_t)out % 16 == 0 && (uintptr_t)weight % 16 == 0 && n <= 4 * 1024 * 4;
  cudaStream_t st = (cudaStream_t)stream;
  if (vec && n <= 1024 && (int64_t)n_tok * groups >= 1024) {
    const int64_t jobs = (int64_t)n_tok * groups;
    SEQ_DISPATCH_DTYPE(dtype, (gated_group_norm_warp_kernel<T><<<(unsigned)((jobs + 7) / 8), 256, 0, st>>>(
                                  x, (const T *)gate, gate_ld, weight, (T *)out, out_ld, out_scale, cols, groups, eps, gate_act, gate_first, jobs)));
    return launch_status();
  }
  if (vec) {
    const int items = n / 4;                                    // vector items per row
    int th = 64;
    while (th < 1024 && th * 4 < items) th *= 2;               // up to four items per thread, up to 1024 threads
    if (n_tok <= 64) while (th < 1024 && th < items) th *= 2;   // short batches: one item per thread where possible
    SEQ_DISPATCH_DTYPE(dtype, (gated_group_norm_kernel<T, 4, 4><<<dim3(n_tok, groups), th, 0, st>>>(
                                  x, (const T *)gate, gate_ld, weight, (T *)out, out_ld, out_scale, cols, groups, eps, gate_act, gate_first)));
    return launch_status();
  }
  const int th = n >= 1024 ? 256 : (n >= 256 ? 128 : 64);
  SEQ_DISPATCH_DTYPE(dtype, (gated_group_norm_kernel<T, 1, 1><<<dim3(n_tok, groups), th, 0, st>>>(
                                x, (const T *)gate, gate_ld, weight, (T *)out, out_ld, out_scale, cols, groups, eps, gate_act, gate_first)));
  return launch_status();
}

extern "C" int mrs_seq_glu_join(const void *x, void *out, int dtype, int n_tok, int half, const mrs_seq_glu_rule *rule, int64_t stream) {
  if (n_tok <= 0 || half <= 0) return 0;
  if (!rule) return -2;
  const int vec = half % 4 == 0 && (uintptr_t)x % 16 == 0 && (uintptr_t)out % 16 == 0;
  const int per = vec ? 1024 : 256, by = (half + per - 1) / per;
  SEQ_DISPATCH_DTYPE(dtype, (glu_split_kernel<T><<<dim3(n_tok, by < 64 ? by : 64), 256, 0, (cudaStream_t)stream>>>(
                                (const T *)x, (T *)out, half, *rule, vec)));
  return launch_status();
}

extern "C" int mrs_seq_glu_split(const void *x, void *out, int dtype, int n_tok, int half, int act, int64_t stream) {
  const mrs_seq_glu_rule rule = {act, 0.0f, 0.0f, 0.0f};
  return mrs_seq_glu_join(x, out, dtype, n_tok, half, &rule, stream);
}

// gate = lower + (1 - lower) * sigmoid(raw + bias), f32
template <typename T>
__global__ void bounded_gate_kernel(const T *__restrict__ raw, int64_t raw_ld, const float *__restrict__ bias, const float *__restrict__ lower,
                                    int cols, float *__restrict__ gate) {
  const int t = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < cols; c += gridDim.y * blockDim.x) {
    const float lo = lower ? lower[c] : 0.0f;
    gate[(int64_t)t * cols + c] = lo + (1.0f - lo) * seq::sigmoid_f(seq::to_f32<T>(raw[(int64_t)t * raw_ld + c]) + (bias ? bias[c] : 0.0f));
  }
}

extern "C" int mrs_seq_bounded_gate(const void *raw, int64_t raw_ld, int dtype, const float *bias, const float *lower, int n_tok, int cols,
                                    float *gate, int64_t stream) {
  if (n_tok <= 0 || cols <= 0) return 0;
  const int by = (cols + 255) / 256;
  SEQ_DISPATCH_DTYPE(dtype, (bounded_gate_kernel<T><<<dim3(n_tok, by < 64 ? by : 64), 256, 0, (cudaStream_t)stream>>>(
                                (const T *)raw, raw_ld, bias, lower, cols, gate)));
  return launch_status();
}

// gate = sigmoid(raw + bias)^power = exp(power * log_sigmoid(raw + bias)), f32; the logarithm is formed without cancellation
template <typename T>
__global__ void power_gate_kernel(const T *__restrict__ raw, int64_t raw_ld, const float *__restrict__ bias, float power, int cols,
                                  float *__restrict__ gate) {
  const int t = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < cols; c += gridDim.y * blockDim.x) {
    const float z = seq::to_f32<T>(raw[(int64_t)t * raw_ld + c]) + (bias ? bias[c] : 0.0f);
    const float log_sig = fminf(z, 0.0f) - log1pf(expf(-fabsf(z)));
    gate[(int64_t)t * cols + c] = expf(power * log_sig);
  }
}

extern "C" int mrs_seq_power_gate(const void *raw, int64_t raw_ld, int dtype, const float *bias, float power, int n_tok, int cols,
                                  float *gate, int64_t stream) {
  if (n_tok <= 0 || cols <= 0) return 0;
  const int by = (cols + 255) / 256;
  SEQ_DISPATCH_DTYPE(dtype, (power_gate_kernel<T><<<dim3(n_tok, by < 64 ? by : 64), 256, 0, (cudaStream_t)stream>>>(
                                (const T *)raw, raw_ld, bias, power, cols, gate)));
  return launch_status();
}

extern "C" int mrs_seq_activate_cols(void *x, int64_t ld, int dtype, int n_tok, int cols, int act, int64_t stream) {
  if (n_tok <= 0 || cols <= 0) return 0;
  const int vec = cols % 4 == 0 && ld % 4 == 0 && (uintptr_t)x % 16 == 0;
  const int per = vec ? 1024 : 256, by = (cols + per - 1) / per;
  SEQ_DISPATCH_DTYPE(dtype, (activate_cols_kernel<T><<<dim3(n_tok, by < 64 ? by : 64), 256, 0, (cudaStream_t)stream>>>((T *)x, ld, cols, act, vec)));
  return launch_status();
}
