// window_attn.cu — softmax attention over a paged cache: RMS norm of queries and keys (per head, or over the whole
// projection), optional rotary positions on part of every head, a sliding window (or full causal reach) that may keep
// the first tokens of the sequence in sight, an optional per-head sink in the softmax denominator, grouped key/value
// heads, values that may be the unnormed keys, and key / value head sizes that need not match.  The new tokens' keys and values are stored first; the attention kernel then reads
// every key of a query, old or new, from the pages — one code path for a prompt portion and for a decoded token.
#include "seq_common.cuh"

namespace seq {

// Query / key preparation, one CTA per token.  Phase 1: sums of squares per head (one warp per q or k head).  Phase 2,
// again one warp per head: the RMS norm (per head with weights shared by the heads, or over the whole projection at
// once with one weight per element), the rotation of the first rot_dims entries in pairs (i, i + rot_dims / 2) by the
// step's cos / sin table, q and k rewritten in place, k stored to its cache slot; values stored from their own
// projection or — v == NULL — from the keys as they were projected (read before the key is rewritten).
template <typename T>
__global__ void attention_prepare_kernel(const mrs_seq_attn_prepare_args a) {
  extern __shared__ float ss[];   // [heads + kv_heads] sums of squares
  const int t = blockIdx.x, lane = threadIdx.x & 31, wib = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int heads = a.heads, kv_heads = a.kv_heads, dk = a.dk, dv = a.dv;
  T *q = (T *)a.q + (int64_t)t * a.q_ld, *k = (T *)a.k + (int64_t)t * a.k_ld;
  const int64_t slot = a.slot_of_tok[t];
  if (a.norm_mode != MRS_SEQ_QK_NORM_NONE) {
    for (int job = wib; job < heads + kv_heads; job += nw) {
      const T *src = job < heads ? q + job * dk : k + (job - heads) * dk;
      float s = 0.0f;
      for (int d = lane; d < dk; d += 32) {
        const float x = to_f32<T>(src[d]);
        s = fmaf(x, x, s);
      }
      s = warp_sum(s);
      if (lane == 0) ss[job] = s;
    }
    __syncthreads();
  }
  float inv_q_all = 1.0f, inv_k_all = 1.0f;
  if (a.norm_mode == MRS_SEQ_QK_NORM_WHOLE) {
    float sq = 0.0f, sk = 0.0f;
    for (int h = 0; h < heads; h++) sq += ss[h];
    for (int h = 0; h < kv_heads; h++) sk += ss[heads + h];
    inv_q_all = rsqrtf_exact(sq / (float)(heads * dk) + a.eps);
    inv_k_all = rsqrtf_exact(sk / (float)(kv_heads * dk) + a.eps);
  }
  const int half = a.cos_sin ? a.rot_dims / 2 : 0;
  const float2 *cs = (const float2 *)a.cos_sin + (int64_t)t * half;
  for (int job = wib; job < heads + 2 * kv_heads; job += nw) {
    if (job < heads + kv_heads) {
      const bool is_q = job < heads;
      const int hh = is_q ? job : job - heads;
      T *src = is_q ? q + hh * dk : k + hh * dk;
      const float *w = is_q ? a.q_norm_w : a.k_norm_w;
      float inv = 1.0f;
      if (a.norm_mode == MRS_SEQ_QK_NORM_HEAD) inv = rsqrtf_exact(ss[job] / (float)dk + a.eps);
      else if (a.norm_mode == MRS_SEQ_QK_NORM_WHOLE) { inv = is_q ? inv_q_all : inv_k_all; w += hh * dk; }
      const bool normed = a.norm_mode != MRS_SEQ_QK_NORM_NONE;
      T *cached = (!is_q && slot >= 0) ? (T *)a.k_cache + (slot * kv_heads + hh) * dk : nullptr;
      if (!is_q && a.v == nullptr) {      // the values are the keys as projected
        if (slot >= 0) {
          T *vc = (T *)a.v_cache + (slot * kv_heads + hh) * dv;
          for (int d = lane; d < dk; d += 32) vc[d] = src[d];
        }
        __syncwarp();
      }
      for (int i = lane; i < half; i += 32) {          // rotated pairs
        const float u = normed ? to_f32<T>(src[i]) * inv * w[i] : to_f32<T>(src[i]);
        const float v = normed ? to_f32<T>(src[i + half]) * inv * w[i + half] : to_f32<T>(src[i + half]);
        const float2 c = cs[i];
        const T ru = from_f32<T>(u * c.x - v * c.y), rv = from_f32<T>(v * c.x + u * c.y);
        src[i] = ru;
        src[i + half] = rv;
        if (cached) { cached[i] = ru; cached[i + half] = rv; }
      }
      for (int d = 2 * half + lane; d < dk; d += 32) {  // the rest passes
        const T r = normed ? from_f32<T>(to_f32<T>(src[d]) * inv * w[d]) : src[d];
        src[d] = r;
        if (cached) cached[d] = r;
      }
    } else if (slot >= 0 && a.v != nullptr) {
      const int hh = job - heads - kv_heads;
      const T *src = (const T *)a.v + (int64_t)t * a.v_ld + hh * dv;
      T *dst = (T *)a.v_cache + (slot * kv_heads + hh) * dv;
      for (int d = lane; d < dv; d += 32) dst[d] = src[d];
    }
  }
}

// cos_sin[t][i] = mag * (cos, sin)(pos[t] * freq[i]): the angle, and its reduction, in double — positions in the thousands
// times a frequency near one leave no digits to spare in f32
__global__ void rotation_table_kernel(const int32_t *__restrict__ pos_of_tok, const double *__restrict__ freq, int n_tok, int half,
                                      float mag, float2 *__restrict__ cos_sin) {
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_tok * half) return;
  const int t = e / half, i = e % half;
  double s, c;
  sincos((double)pos_of_tok[t] * freq[i], &s, &c);
  cos_sin[e] = make_float2((float)(c * (double)mag), (float)(s * (double)mag));
}

// Cache row of entry j of a sequence: token position j through the page table, or — pool > 0 — the averaged entry of block j,
// which sits behind the token rows: per page as many entries as blocks can START in a page, a block at the page of its
// first position.
__device__ __forceinline__ int64_t key_row(const int32_t *table, int j, int pool, int page_size, int per_page, int64_t pool_base) {
  if (pool <= 0) return (int64_t)table[j / page_size] * page_size + j % page_size;
  const int page = (j * pool) / page_size, first = (page * page_size + pool - 1) / pool;
  return pool_base + (int64_t)table[page] * per_page + (j - first);
}
template <typename T> __device__ __forceinline__ void store_out(T *out, int64_t at, float v, int as_f32) {
  if (as_f32) ((float *)out)[at] = v;
  else out[at] = from_f32<T>(v);
}

// One warp per (token, head).  32 keys per round: lane j scores key j against the whole query (held in shared
// memory as f32, pre-scaled), the round's maximum and sum go through the warp, then every lane accumulates its
// value columns over the round's keys.  Softmax statistics and the output accumulate in f32.
template <typename T, int MAX_VCOLS>   // MAX_VCOLS * 32 >= value head size
__global__ void __launch_bounds__(128) window_attention_kernel(const T *__restrict__ q, int64_t q_ld, const T *__restrict__ k_cache,
                                                               const T *__restrict__ v_cache, int heads, int kv_heads, int dk, int dv,
                                                               float scale, int window, int keep_first, const float *__restrict__ sink,
                                                               const int32_t *__restrict__ pages,
                                                               int pages_ld, int page_size, const int32_t *__restrict__ seq_of_tok,
                                                               const int32_t *__restrict__ pos_of_tok, const int32_t *__restrict__ tok_index,
                                                               int n_tok, T *__restrict__ out, int64_t out_ld, float out_scale, int64_t k_row,
                                                               int64_t v_row, int pool, int64_t pool_base, int v_shared, int out_f32, int64_t out_head) {
  extern __shared__ __align__(16) float qsm[];   // [warps][dk]
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int64_t job = (int64_t)blockIdx.x * (blockDim.x >> 5) + wib;
  if (job >= (int64_t)n_tok * heads) return;
  const int ti = (int)(job / heads), t = tok_index ? tok_index[ti] : ti, h = (int)(job % heads), g = h / (heads / kv_heads);
  const int s = seq_of_tok[t], pos = pos_of_tok[t];
  float *qv = qsm + wib * dk;
  for (int d = lane; d < dk; d += 32) qv[d] = to_f32<T>(q[(int64_t)t * q_ld + h * dk + d]) * scale;
  __syncwarp();
  const int32_t *table = pages + (int64_t)s * pages_ld;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  float m = -INFINITY, l = 0.0f, acc[MAX_VCOLS];
#pragma unroll
  for (int c = 0; c < MAX_VCOLS; c++) acc[c] = 0.0f;
  // entries before the window: the kept first keys [0, kept), or one averaged entry per whole block of `pool` positions
  const int kept = pool > 0 ? lo / pool : min(keep_first, lo);
  const int kept_rounds = (kept + 31) / 32, rounds = kept_rounds + (pos - lo) / 32 + 1;
  const int gv = v_shared ? 0 : g, per_page = pool > 0 ? (page_size + pool - 1) / pool : 0;
  for (int r = 0; r < rounds; r++) {
    const int j0 = r < kept_rounds ? r * 32 : lo + (r - kept_rounds) * 32, jend = r < kept_rounds ? kept : pos + 1;
    const int j = j0 + lane;
    float sc = -INFINITY;
    int64_t slot = 0;
    if (j < jend) {
      slot = key_row(table, j, r < kept_rounds ? pool : 0, page_size, per_page, pool_base);
      const T *kr = k_cache + slot * k_row + g * dk;
      float a0 = 0.0f, a1 = 0.0f;
      int d = 0;
      for (; d + 1 < dk; d += 2) {
        a0 = fmaf(qv[d], to_f32<T>(kr[d]), a0);
        a1 = fmaf(qv[d + 1], to_f32<T>(kr[d + 1]), a1);
      }
      if (d < dk) a0 = fmaf(qv[d], to_f32<T>(kr[d]), a0);
      sc = a0 + a1;
    }
    const float m_new = fmaxf(m, warp_max(sc));      // the round always holds key j0 < jend: m_new is finite
    const float p = j < jend ? expf(sc - m_new) : 0.0f;
    const float corr = expf(m - m_new);               // exp(-inf) = 0 on the first round
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < MAX_VCOLS; c++) acc[c] *= corr;
    const int n = min(32, jend - j0);
    for (int i = 0; i < n; i++) {
      const float pi = __shfl_sync(0xffffffffu, p, i);
      const int64_t si = __shfl_sync(0xffffffffu, slot, i);
      const T *vr = v_cache + si * v_row + gv * dv;
#pragma unroll
      for (int c = 0; c < MAX_VCOLS; c++)
        if (c * 32 + lane < dv) acc[c] = fmaf(pi, to_f32<T>(vr[c * 32 + lane]), acc[c]);
    }
    m = m_new;
  }
  if (sink) l += expf(sink[h] - m);                  // a key without a value; its score is not scaled
  const float inv = out_scale / l;
#pragma unroll
  for (int c = 0; c < MAX_VCOLS; c++)
    if (c * 32 + lane < dv) store_out<T>(out, (int64_t)t * out_ld + h * out_head + c * 32 + lane, acc[c] * inv, out_f32);
}

// The same computation laid out for speed when the head sizes allow vector loads (dk a multiple of 8 and dv even):
// one CTA of SPLIT warps per (token, head); the warps take the window's 32-key rounds in turn and their partial
// (max, sum, output) triples are merged through shared memory.  Keys are read 16 bytes at a time, values two columns
// per lane.
template <typename T, int VPAIRS, int SPLIT>   // VPAIRS * 64 >= dv
__global__ void __launch_bounds__(SPLIT * 32) window_attention_vec_kernel(
    const T *__restrict__ q, int64_t q_ld, const T *__restrict__ k_cache, const T *__restrict__ v_cache, int heads, int kv_heads, int dk, int dv,
    float scale, int window, int keep_first, const float *__restrict__ sink, const int32_t *__restrict__ pages, int pages_ld, int page_size,
    const int32_t *__restrict__ seq_of_tok, const int32_t *__restrict__ pos_of_tok, const int32_t *__restrict__ tok_index, T *__restrict__ out,
    int64_t out_ld, float out_scale, int64_t k_row, int64_t v_row, int pool, int64_t pool_base, int v_shared, int out_f32, int64_t out_head) {
  extern __shared__ __align__(16) float sm[];   // q [dk] | per warp: m, l, acc [VPAIRS * 64]
  const int lane = threadIdx.x & 31, wib = threadIdx.x >> 5;
  const int ti = blockIdx.x / heads, h = blockIdx.x % heads, t = tok_index ? tok_index[ti] : ti, g = h / (heads / kv_heads);
  const int s = seq_of_tok[t], pos = pos_of_tok[t];
  float *qv = sm, *part = sm + dk;
  for (int d = threadIdx.x; d < dk; d += SPLIT * 32) qv[d] = to_f32<T>(q[(int64_t)t * q_ld + h * dk + d]) * scale;
  __syncthreads();
  const int32_t *table = pages + (int64_t)s * pages_ld;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  float m = -INFINITY, l = 0.0f;
  float2 acc[VPAIRS];
#pragma unroll
  for (int c = 0; c < VPAIRS; c++) acc[c] = make_float2(0.0f, 0.0f);
  constexpr int N = Vec16<T>::N;
  // entries before the window: the kept first keys [0, kept), or one averaged entry per whole block of `pool` positions
  const int kept = pool > 0 ? lo / pool : min(keep_first, lo);
  const int kept_rounds = (kept + 31) / 32, rounds = kept_rounds + (pos - lo) / 32 + 1;
  const int gv = v_shared ? 0 : g, per_page = pool > 0 ? (page_size + pool - 1) / pool : 0;
  for (int r = wib; r < rounds; r += SPLIT) {
    const int j0 = r < kept_rounds ? r * 32 : lo + (r - kept_rounds) * 32, jend = r < kept_rounds ? kept : pos + 1;
    const int j = j0 + lane;
    float sc = -INFINITY;
    int64_t slot = 0;
    if (j < jend) {
      slot = key_row(table, j, r < kept_rounds ? pool : 0, page_size, per_page, pool_base);
      const T *kr = k_cache + slot * k_row + g * dk;
      float a0 = 0.0f, a1 = 0.0f;
      int d = 0;
#pragma unroll 4
      for (; d + 2 * N <= dk; d += 2 * N) {
        a0 += dot16<T>(qv + d, kr + d);
        a1 += dot16<T>(qv + d + N, kr + d + N);
      }
      for (; d < dk; d += N) a0 += dot16<T>(qv + d, kr + d);
      sc = a0 + a1;
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float p = j < jend ? expf(sc - m_new) : 0.0f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < VPAIRS; c++) { acc[c].x *= corr; acc[c].y *= corr; }
    const int n = min(32, jend - j0);
    // eight keys per pass: their value rows are fetched together, so the loads overlap instead of queueing behind the
    // shuffles that carry each key's slot
    constexpr int KPP = VPAIRS > 4 ? 4 : 8;       // keys per pass: fewer for wide values, whose rows fill the registers sooner
    for (int i0 = 0; i0 < n; i0 += KPP) {
      float pi[KPP];
      float2 vv[KPP][VPAIRS];
#pragma unroll
      for (int u = 0; u < KPP; u++) {
        const int i = min(i0 + u, 31);
        const float pu = __shfl_sync(0xffffffffu, p, i);
        pi[u] = i0 + u < n ? pu : 0.0f;
        const int64_t si = __shfl_sync(0xffffffffu, slot, i);
        const T *vr = v_cache + si * v_row + gv * dv;              // a lane past n carries slot 0: a valid row, weight 0
#pragma unroll
        for (int c = 0; c < VPAIRS; c++)
          vv[u][c] = c * 64 + 2 * lane < dv ? load2<T>(vr + c * 64 + 2 * lane) : make_float2(0.0f, 0.0f);
      }
#pragma unroll
      for (int u = 0; u < KPP; u++)
#pragma unroll
        for (int c = 0; c < VPAIRS; c++) {
          acc[c].x = fmaf(pi[u], vv[u][c].x, acc[c].x);
          acc[c].y = fmaf(pi[u], vv[u][c].y, acc[c].y);
        }
    }
    m = m_new;
  }
  float *mine = part + wib * (2 + VPAIRS * 64);
  if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
  for (int c = 0; c < VPAIRS; c++) { mine[2 + c * 64 + 2 * lane] = acc[c].x; mine[2 + c * 64 + 2 * lane + 1] = acc[c].y; }
  __syncthreads();
  float mx = -INFINITY;
  for (int w = 0; w < SPLIT; w++) mx = fmaxf(mx, part[w * (2 + VPAIRS * 64)]);
  float lsum = 0.0f;
  for (int w = 0; w < SPLIT; w++) {
    const float mw = part[w * (2 + VPAIRS * 64)];
    if (mw != -INFINITY) lsum += part[w * (2 + VPAIRS * 64) + 1] * expf(mw - mx);
  }
  if (sink) lsum += expf(sink[h] - mx);              // warp 0 always holds a key: mx is finite
  const float inv = out_scale / lsum;
  for (int c = threadIdx.x; c < dv; c += SPLIT * 32) {
    float o = 0.0f;
    for (int w = 0; w < SPLIT; w++) {
      const float mw = part[w * (2 + VPAIRS * 64)];
      if (mw != -INFINITY) o = fmaf(part[w * (2 + VPAIRS * 64) + 2 + c], expf(mw - mx), o);
    }
    store_out<T>(out, (int64_t)t * out_ld + h * out_head + c, o * inv, out_f32);
  }
}

template <typename T>
__global__ void scale_rows_kernel(T *__restrict__ x, int64_t ld, int cols, float scale) {
  T *row = x + (int64_t)blockIdx.x * ld;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) row[c] = from_f32<T>(to_f32<T>(row[c]) * scale);
}

}  // namespace seq

using namespace seq;

extern "C" int mrs_seq_attention_prepare(const mrs_seq_attn_prepare_args *args, int64_t stream) {
  const mrs_seq_attn_prepare_args &a = *args;
  if (a.n_tok <= 0) return 0;
  if (a.heads <= 0 || a.kv_heads <= 0 || a.dk <= 0 || a.dv <= 0 || !a.q || !a.k || !a.slot_of_tok) return -2;
  if (a.norm_mode != MRS_SEQ_QK_NORM_NONE && (!a.q_norm_w || !a.k_norm_w)) return -2;
  if (a.v == nullptr && a.dv != a.dk) return -2;
  if (a.cos_sin && (a.rot_dims < 2 || a.rot_dims % 2 || a.rot_dims > a.dk)) return -2;
  const int jobs = a.heads + 2 * a.kv_heads, warps = jobs < 8 ? jobs : 8;
  const size_t bytes = (size_t)(a.heads + a.kv_heads) * sizeof(float);
  SEQ_DISPATCH_DTYPE(a.dtype, (attention_prepare_kernel<T><<<a.n_tok, warps * 32, bytes, (cudaStream_t)stream>>>(a)));
  return launch_status();
}

extern "C" int mrs_seq_qk_norm_store(void *q, int64_t q_ld, void *k, int64_t k_ld, const void *v, int64_t v_ld, int dtype,
                                     const float *q_norm_w, const float *k_norm_w, float eps, int heads, int kv_heads, int dk, int dv,
                                     void *k_cache, void *v_cache, const int64_t *slot_of_tok, int n_tok, int64_t stream) {
  if (!v) return -2;
  mrs_seq_attn_prepare_args a = {};
  a.q = q; a.k = k; a.v = v; a.q_ld = q_ld; a.k_ld = k_ld; a.v_ld = v_ld;
  a.dtype = dtype; a.norm_mode = (q_norm_w && k_norm_w) ? MRS_SEQ_QK_NORM_HEAD : MRS_SEQ_QK_NORM_NONE;
  a.q_norm_w = q_norm_w; a.k_norm_w = k_norm_w; a.eps = eps;
  a.heads = heads; a.kv_heads = kv_heads; a.dk = dk; a.dv = dv;
  a.k_cache = k_cache; a.v_cache = v_cache; a.slot_of_tok = slot_of_tok; a.n_tok = n_tok;
  return mrs_seq_attention_prepare(&a, stream);
}

extern "C" int mrs_seq_rotation_table(const int32_t *pos_of_tok, const double *freq, int n_tok, int half, float mag, float *cos_sin,
                                      int64_t stream) {
  if (n_tok <= 0 || half <= 0) return 0;
  const int total = n_tok * half;
  rotation_table_kernel<<<(total + 127) / 128, 128, 0, (cudaStream_t)stream>>>(pos_of_tok, freq, n_tok, half, mag, (float2 *)cos_sin);
  return launch_status();
}

extern "C" int mrs_seq_paged_attention(const mrs_seq_paged_attention_args *args, int64_t stream) {
  const mrs_seq_paged_attention_args &a = *args;
  const int n_tok = a.n_tok, heads = a.heads, kv_heads = a.kv_heads, dk = a.dk, dv = a.dv, dtype = a.dtype;
  if (n_tok <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || dv > 1024 || dk > 2048 || a.page_size <= 0) return -2;
  const int keep_first = a.keep_first > 0 ? a.keep_first : 0, pool = a.pool > 0 ? a.pool : 0;
  if (pool > 0 && (a.window <= 0 || keep_first > 0)) return -2;      // averaged blocks lie before a window and replace kept first keys
  cudaStream_t st = (cudaStream_t)stream;
  const int elem = dtype == MRS_SEQ_BF16 ? 2 : 4;
  const int64_t k_row = a.k_row > 0 ? a.k_row : (int64_t)kv_heads * dk, v_row = a.v_row > 0 ? a.v_row : (int64_t)kv_heads * dv;
  const int64_t out_head = a.out_head > 0 ? a.out_head : dv;
  const bool vec = dk % (16 / elem) == 0 && dv % 2 == 0 && dv <= 512 && ((uintptr_t)a.k_cache % 16) == 0 && ((uintptr_t)a.v_cache % 8) == 0 &&
                   k_row % (16 / elem) == 0 && v_row % 2 == 0;
  if (vec) {
    constexpr int SPLIT = 8;
#define SEQ_ATTN_VEC(VP)                                                                                                         \
  window_attention_vec_kernel<T, VP, SPLIT><<<(unsigned)n_tok * heads, SPLIT * 32, (dk + SPLIT * (2 + VP * 64)) * sizeof(float), st>>>( \
      (const T *)a.q, a.q_ld, (const T *)a.k_cache, (const T *)a.v_cache, heads, kv_heads, dk, dv, a.scale, a.window, keep_first, a.sink,  \
      a.pages, a.pages_ld, a.page_size, a.seq_of_tok, a.pos_of_tok, a.tok_index, (T *)a.out, a.out_ld, a.out_scale, k_row, v_row, pool,     \
      a.pool_base, a.v_shared, a.out_f32, out_head)
    SEQ_DISPATCH_DTYPE(dtype, {
      if (dv <= 64) SEQ_ATTN_VEC(1);
      else if (dv <= 128) SEQ_ATTN_VEC(2);
      else if (dv <= 256) SEQ_ATTN_VEC(4);
      else SEQ_ATTN_VEC(8);
    });
#undef SEQ_ATTN_VEC
    return launch_status();
  }
  const int warps = 4;
  const int64_t jobs = (int64_t)n_tok * heads;
#define SEQ_ATTN_LAUNCH(VC)                                                                                              \
  window_attention_kernel<T, VC><<<(unsigned)((jobs + warps - 1) / warps), warps * 32, warps * dk * sizeof(float), st>>>(  \
      (const T *)a.q, a.q_ld, (const T *)a.k_cache, (const T *)a.v_cache, heads, kv_heads, dk, dv, a.scale, a.window, keep_first, a.sink, \
      a.pages, a.pages_ld, a.page_size, a.seq_of_tok, a.pos_of_tok, a.tok_index, n_tok, (T *)a.out, a.out_ld, a.out_scale, k_row, v_row, pool, \
      a.pool_base, a.v_shared, a.out_f32, out_head)
  SEQ_DISPATCH_DTYPE(dtype, {
    if (dv <= 64) SEQ_ATTN_LAUNCH(2);
    else if (dv <= 128) SEQ_ATTN_LAUNCH(4);
    else if (dv <= 256) SEQ_ATTN_LAUNCH(8);
    else if (dv <= 512) SEQ_ATTN_LAUNCH(16);
    else SEQ_ATTN_LAUNCH(32);
  });
#undef SEQ_ATTN_LAUNCH
  return launch_status();
}

extern "C" int mrs_seq_window_attention(const void *q, int64_t q_ld, const void *k_cache, const void *v_cache, int dtype, int heads,
                                        int kv_heads, int dk, int dv, float scale, int window, const int32_t *pages, int pages_ld,
                                        int page_size, const int32_t *seq_of_tok, const int32_t *pos_of_tok, const int32_t *tok_index,
                                        int n_tok, void *out, int64_t out_ld, float out_scale, int64_t stream) {
  mrs_seq_paged_attention_args a = {};
  a.q = q; a.q_ld = q_ld; a.k_cache = k_cache; a.v_cache = v_cache;
  a.dtype = dtype; a.heads = heads; a.kv_heads = kv_heads; a.dk = dk; a.dv = dv;
  a.scale = scale; a.window = window;
  a.pages = pages; a.pages_ld = pages_ld; a.page_size = page_size;
  a.seq_of_tok = seq_of_tok; a.pos_of_tok = pos_of_tok; a.tok_index = tok_index; a.n_tok = n_tok;
  a.out = out; a.out_ld = out_ld; a.out_scale = out_scale;
  return mrs_seq_paged_attention(&a, stream);
}

extern "C" int mrs_seq_scale_rows(void *x, int64_t ld, int dtype, int rows, int cols, float scale, int64_t stream) {
  if (rows <= 0 || cols <= 0) return 0;
  SEQ_DISPATCH_DTYPE(dtype, (scale_rows_kernel<T><<<rows, 256, 0, (cudaStream_t)stream>>>((T *)x, ld, cols, scale)));
  return launch_status();
}
