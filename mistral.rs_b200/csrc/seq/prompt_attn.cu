// prompt_attn.cu — tensor-core attention of the long portions of a step (a prompt's first portion or a later one) for
// layers whose softmax may have a sink and whose window may keep the first tokens in sight.  Queries are the portion's
// fresh rows; keys and values — the portion's own and everything the sequence cached before — are read from the pages,
// where the preparation kernel has just stored them, so one kernel serves whole prompts and prompts cut anywhere.
//
// The tiling is the package's mma.sync prompt kernel (prefill_attn.cu): one CTA = 128 query rows of one (sequence,
// head), 8 warps x 16 rows, Q fragments in registers, K / V tiles of 64 positions through a double-buffered XOR-swizzled
// shared-memory ring (cp.async, 16 bytes at a time, the page looked up per row), S = QK^T and O = PV as m16n8k16 MMAs
// with f32 accumulation, online softmax in f32 on a base-2 exponent.  The key tiles of a query tile are the kept first
// tiles followed by the window's tiles; the denominator ends with the sink's term.
//
// Two further forms of the same loop.  Averaged blocks (pool > 0): instead of kept first keys, the tiles before the window
// hold one averaged key / value row per block of `pool` positions (rows pool_base.. of the same cache tensors, see
// window_attn.cu's key_row); entry b is visible to a query at position i when the block ends at or before i - window.
// Every value head (v_heads > 1): grid.y runs over (value head, query head) pairs — the head's own keys, the given value
// head's values — and the result goes to an f32 matrix [tokens, heads, v_heads * D]; a mixing of softmax weights across
// heads is then a weighted sum of these rows (pooled.cu's mix_heads).
#include "../mma_common.cuh"

#include "../../../include/mrs_b200_seq.h"

namespace seqp {
using namespace mrs;

constexpr int BM = 128, BN = 64, WARPS = 8, THREADS = WARPS * 32;

struct Params {
  const __nv_bfloat16 *q, *k_cache, *v_cache;
  __nv_bfloat16 *o;
  const int32_t *portions;     // [n][4]: first row, rows, positions cached before (past), row of the page table
  const int32_t *pages;
  int pages_ld, page_size;
  int H, KVH;
  int64_t q_ld, o_ld;
  float scale_log2;
  int window, keep_first;      // window <= 0: every earlier position
  const float *sink;
  int pool, per_page;          // pool > 0: averaged blocks before the window; per_page = ceil(page_size / pool)
  int64_t pool_base;
  int v_heads;                 // 1, or the number of value heads when every head is applied to every value head
  int o_f32;                   // the result is f32 [tokens, heads, v_heads * D] (o is then float *)
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1) prompt_attention_kernel(const Params p) {
  using T = __nv_bfloat16;
  constexpr int KSTEPS = D / 16, DT = D / 8, CPR = D / 8, TILE_BYTES = BN * D * 2;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t *sk[2] = {smem, smem + 2 * TILE_BYTES};
  uint8_t *sv[2] = {smem + TILE_BYTES, smem + 3 * TILE_BYTES};

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.z, h = blockIdx.y % p.H, vsel = blockIdx.y / p.H, kvh = h / (p.H / p.KVH);
  const int vh = p.v_heads > 1 ? vsel : kvh;        // the value head this CTA applies the head's weights to
  const int seq0 = p.portions[4 * b], len = p.portions[4 * b + 1], past = p.portions[4 * b + 2];
  const int32_t *table = p.pages + (int64_t)p.portions[4 * b + 3] * p.pages_ld;
  const int total = past + len;                     // positions the sequence holds after this step
  const int ntile_q = (len + BM - 1) / BM;
  const int qt = ntile_q - 1 - (int)blockIdx.x;     // heavy tiles first
  if (qt < 0) return;
  const int q0 = qt * BM;                           // row inside the portion; its position is past + row
  const T *qg = p.q + (int64_t)seq0 * p.q_ld + (int64_t)h * D;
  T *og = p.o + (int64_t)seq0 * p.o_ld + (int64_t)h * D;
  float *ogf = (float *)p.o + (int64_t)seq0 * p.o_ld + ((int64_t)h * p.v_heads + vsel) * D;

  // key tiles of this query tile: the kept first positions that lie before the window's first tile, then the window
  const int kv_end = min(total, past + q0 + BM);
  const int win_begin = p.window > 0 ? max(0, past + q0 - p.window + 1) / BN * BN : 0;
  // entries before the window: kept first positions, or averaged blocks (as many as the tile's last query sees)
  const int kept_end = p.pool > 0 ? max(0, kv_end - p.window) / p.pool : min(p.keep_first, win_begin);
  const int kept_tiles = (kept_end + BN - 1) / BN;                  // kept_tiles * BN <= win_begin: no key twice
  const int nt = kept_tiles + (kv_end - win_begin + BN - 1) / BN;
  auto tile_start = [&](int t) { return t < kept_tiles ? t * BN : win_begin + (t - kept_tiles) * BN; };

  auto load_tile = [&](int t, int buf) {
    const int t0 = tile_start(t);
    for (int c = tid; c < BN * CPR; c += THREADS) {
      const int row = c / CPR, ch = c % CPR;
      const int j = t0 + row;
      const bool averaged = p.pool > 0 && t < kept_tiles;
      const bool ok = j < (averaged ? kept_end : kv_end);
      const int jj = ok ? j : 0;
      int64_t slot;
      if (averaged) {
        const int page = (jj * p.pool) / p.page_size, first = (page * p.page_size + p.pool - 1) / p.pool;
        slot = p.pool_base + (int64_t)table[page] * p.per_page + (jj - first);
      } else {
        slot = (int64_t)table[jj / p.page_size] * p.page_size + jj % p.page_size;
      }
      cp_async16(sk[buf] + tile_off<D>(row, ch), p.k_cache + (slot * p.KVH + kvh) * D + ch * 8, ok);
      cp_async16(sv[buf] + tile_off<D>(row, ch), p.v_cache + (slot * p.KVH + vh) * D + ch * 8, ok);
    }
    cp_async_commit();
  };

  uint32_t qa[KSTEPS][4];
  {
    uint8_t *sq = sk[1];   // 128 rows x D: buffer 1 of K and V, free until the second tile arrives
    for (int c = tid; c < BM * CPR; c += THREADS) {
      const int row = c / CPR, ch = c % CPR;
      const bool ok = q0 + row < len;
      cp_async16(sq + tile_off<D>(row, ch), qg + (int64_t)(ok ? q0 + row : 0) * p.q_ld + ch * 8, ok);
    }
    cp_async_commit();
    load_tile(0, 0);
    cp_async_wait<1>();
    __syncthreads();
    const int r = warp * 16 + (lane & 15);
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) ldsm_x4(smem_u32(sq + tile_off<D>(r, 2 * ks + (lane >> 4))), qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3]);
    __syncthreads();
  }

  float oacc[DT][4];
#pragma unroll
  for (int i = 0; i < DT; i++) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_a = q0 + warp * 16 + (lane >> 2);   // this thread's accumulator rows (inside the portion): row_a, row_a + 8

  for (int t = 0; t < nt; t++) {
    const int buf = t & 1;
    if (t + 1 < nt) load_tile(t + 1, buf ^ 1);
    else cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int t0 = tile_start(t);

    float sacc[BN / 8][4];
#pragma unroll
    for (int j = 0; j < BN / 8; j++) { sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ks++) {
#pragma unroll
      for (int jp = 0; jp < BN / 16; jp++) {
        const int row = 16 * jp + (lane & 7) + ((lane >> 4) << 3);
        const int ch = 2 * ks + ((lane >> 3) & 1);
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_u32(sk[buf] + tile_off<D>(row, ch)), b0, b1, b2, b3);
        mma16816<T>(sacc[2 * jp], qa[ks], b0, b1);
        mma16816<T>(sacc[2 * jp + 1], qa[ks], b2, b3);
      }
    }

    const bool need_mask = p.window > 0 || t0 + BN > kv_end || t0 + BN - 1 > past + q0 + warp * 16;
    float mx[2] = {m_run[0], m_run[1]};
#pragma unroll
    for (int j = 0; j < BN / 8; j++) {
#pragma unroll
      for (int e = 0; e < 4; e++) {
        float s = sacc[j][e] * p.scale_log2;
        if (need_mask) {
          const int col = t0 + 8 * j + 2 * (lane & 3) + (e & 1);
          const int row = past + row_a + ((e >> 1) << 3);          // the query's position
          bool ok;
          if (p.pool > 0 && t < kept_tiles) ok = (col + 1) * p.pool - 1 <= row - p.window;        // the block ends at or before row - window
          else ok = col < total && col <= row && (p.window <= 0 || row - col < p.window || col < p.keep_first);
          if (!ok) s = -INFINITY;
        }
        sacc[j][e] = s;
        mx[e >> 1] = fmaxf(mx[e >> 1], s);
      }
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    }
    float corr[2], rs[2] = {0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 2; r++) {
      corr[r] = (mx[r] == -INFINITY) ? 1.f : exp2f(m_run[r] - mx[r]);
      m_run[r] = mx[r];
    }
    uint32_t pa[BN / 16][4];
#pragma unroll
    for (int j = 0; j < BN / 8; j++) {
      const float p0 = (mx[0] == -INFINITY) ? 0.f : exp2f(sacc[j][0] - mx[0]);
      const float p1 = (mx[0] == -INFINITY) ? 0.f : exp2f(sacc[j][1] - mx[0]);
      const float p2 = (mx[1] == -INFINITY) ? 0.f : exp2f(sacc[j][2] - mx[1]);
      const float p3 = (mx[1] == -INFINITY) ? 0.f : exp2f(sacc[j][3] - mx[1]);
      rs[0] += p0 + p1; rs[1] += p2 + p3;
      pa[j >> 1][(j & 1) * 2] = pack2<T>(p0, p1);
      pa[j >> 1][(j & 1) * 2 + 1] = pack2<T>(p2, p3);
    }
#pragma unroll
    for (int r = 0; r < 2; r++) l_run[r] = l_run[r] * corr[r] + rs[r];
#pragma unroll
    for (int i = 0; i < DT; i++) { oacc[i][0] *= corr[0]; oacc[i][1] *= corr[0]; oacc[i][2] *= corr[1]; oacc[i][3] *= corr[1]; }

#pragma unroll
    for (int kk = 0; kk < BN / 16; kk++) {
#pragma unroll
      for (int dp = 0; dp < DT / 2; dp++) {
        const int row = 16 * kk + (lane & 7) + (((lane >> 3) & 1) << 3);
        const int ch = 2 * dp + (lane >> 4);
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_u32(sv[buf] + tile_off<D>(row, ch)), b0, b1, b2, b3);
        mma16816<T>(oacc[2 * dp], pa[kk], b0, b1);
        mma16816<T>(oacc[2 * dp + 1], pa[kk], b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; r++) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    // the sink: a key without a value whose score is not scaled; m_run is in base-2 units
    if (p.sink) l_run[r] += exp2f(p.sink[h] * 1.4426950408889634f - m_run[r]);
  }
  const float inv0 = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv1 = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
  for (int i = 0; i < DT; i++) {
    const int col = 8 * i + 2 * (lane & 3);
    if (p.o_f32) {
      if (row_a < len) *(float2 *)(ogf + (int64_t)row_a * p.o_ld + col) = make_float2(oacc[i][0] * inv0, oacc[i][1] * inv0);
      if (row_a + 8 < len) *(float2 *)(ogf + (int64_t)(row_a + 8) * p.o_ld + col) = make_float2(oacc[i][2] * inv1, oacc[i][3] * inv1);
      continue;
    }
    if (row_a < len) *(uint32_t *)(og + (int64_t)row_a * p.o_ld + col) = pack2<T>(oacc[i][0] * inv0, oacc[i][1] * inv0);
    if (row_a + 8 < len) *(uint32_t *)(og + (int64_t)(row_a + 8) * p.o_ld + col) = pack2<T>(oacc[i][2] * inv1, oacc[i][3] * inv1);
  }
}

template <int D>
static int launch(const Params &p, int n, int longest, cudaStream_t st) {
  auto kern = prompt_attention_kernel<D>;
  const size_t bytes = 4 * (size_t)BN * D * 2;
  static bool raised = false;
  if (!raised) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
    raised = true;
  }
  kern<<<dim3((longest + BM - 1) / BM, p.H * p.v_heads, n), THREADS, bytes, st>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace seqp

extern "C" int mrs_seq_prompt_attention(const void *q, int64_t q_ld, const void *k_cache, const void *v_cache, void *out, int64_t out_ld,
                                        const int32_t *portions, int n_portions, int longest, const int32_t *pages, int pages_ld,
                                        int page_size, int heads, int kv_heads, int d, float scale, int window, int keep_first,
                                        const float *sink, int64_t stream) {
  return mrs_seq_prompt_attention_pooled(q, q_ld, k_cache, v_cache, out, out_ld, portions, n_portions, longest, pages, pages_ld, page_size, heads,
                                         kv_heads, d, scale, window, keep_first, sink, 0, 0, 0, stream);
}

extern "C" int mrs_seq_prompt_attention_pooled(const void *q, int64_t q_ld, const void *k_cache, const void *v_cache, void *out, int64_t out_ld,
                                               const int32_t *portions, int n_portions, int longest, const int32_t *pages, int pages_ld,
                                               int page_size, int heads, int kv_heads, int d, float scale, int window, int keep_first,
                                               const float *sink, int pool, int64_t pool_base, int every_value_head, int64_t stream) {
  if (n_portions <= 0 || longest <= 0) return 0;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || (d != 64 && d != 128) || !portions || !pages || page_size <= 0) return -2;
  if (pool > 0 && (window <= 0 || keep_first > 0)) return -2;
  if ((int64_t)heads * (every_value_head ? kv_heads : 1) > 65535) return -2;
  if ((q_ld | out_ld) % 8 || (((uintptr_t)q | (uintptr_t)k_cache | (uintptr_t)v_cache | (uintptr_t)out) & 15)) return -3;
  seqp::Params p = {};
  p.q = (const __nv_bfloat16 *)q; p.k_cache = (const __nv_bfloat16 *)k_cache; p.v_cache = (const __nv_bfloat16 *)v_cache;
  p.o = (__nv_bfloat16 *)out;
  p.portions = portions; p.pages = pages; p.pages_ld = pages_ld; p.page_size = page_size;
  p.H = heads; p.KVH = kv_heads; p.q_ld = q_ld; p.o_ld = out_ld;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window; p.keep_first = keep_first > 0 ? keep_first : 0; p.sink = sink;
  p.pool = pool > 0 ? pool : 0; p.per_page = pool > 0 ? (page_size + pool - 1) / pool : 0; p.pool_base = pool_base;
  p.v_heads = every_value_head ? kv_heads : 1;
  p.o_f32 = every_value_head ? 1 : 0;
  return d == 128 ? seqp::launch<128>(p, n_portions, longest, (cudaStream_t)stream) : seqp::launch<64>(p, n_portions, longest, (cudaStream_t)stream);
}
