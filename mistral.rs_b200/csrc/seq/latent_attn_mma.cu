// latent_attn_mma.cu — tensor-core attention over cached latents (the absorbed form of multi-head latent attention)
// for the long portions of a step.  Every head of a token scores the SAME cached rows (one key/value "head" of size
// dk = kv_rank + rot_dim whose values are its first kv_rank columns), so the (token, head) pairs of a portion are the
// rows of one query matrix: row r belongs to token r / heads and sees positions up to that token's.  One CTA takes
// 16 * MT neighbouring rows and walks the key tiles of their window once — a tile of latents, fetched once into shared
// memory (cp.async, 16 bytes at a time, the page looked up per row), serves all heads both as keys and as values.
//
// Per key tile of 64 positions, three phases separated by block barriers:
//   A  S = Q K^T on m16n8k16 MMAs: warp w takes row tile w % MT and 64 / (8 / MT) of the tile's keys; Q fragments come
//      from shared memory at every k-step (dk is a run-time size), scores go to shared memory as f32 in base-2 units;
//   B  online softmax in f32: 256 / rows threads per row mask, exponentiate and sum their columns, keep the row's running
//      maximum and sum in registers, and leave P (bf16) and the row's rescale factor in shared memory;
//   C  O = O * rescale + P V: warp w takes row tile w % MT and one of 8 / MT column groups of the kv_rank output columns
//      (at most 128 columns, 64 accumulator registers), V fragments are transposed loads of the same key tile.
// MT = 4, 2, 1 for kv_rank up to 256, 512, 1024.  bf16 only; dk and kv_rank multiples of 8.
// A decoded token is a portion of one token: its heads are the rows of one tile and the window's latents are fetched once
// for all of them, where a (token, head) kernel fetches them once per head.
#include "../mma_common.cuh"

#include "../../../include/mrs_b200_seq.h"

namespace seql {
using namespace mrs;

constexpr int BN = 64, WARPS = 8, THREADS = WARPS * 32, SS = BN + 4, PB = BN * 2 + 16, MAX_TILES = 16;

struct Params {
  const __nv_bfloat16 *q, *cache;
  __nv_bfloat16 *o;
  int64_t q_ld, o_ld, cache_row;
  const int32_t *portions;     // [n][4]: first token row, tokens, positions cached before (past), row of the page table; or NULL:
  const int32_t *cu_tok, *past;   // every sequence of the step — tokens cu_tok[b] .. cu_tok[b + 1], past[b] cached before, table row b
  const int32_t *pages;
  int pages_ld, page_size;
  int H, DK, R;
  float scale_log2;
  int window;                  // <= 0: every earlier position
};

template <int MT>
__global__ void __launch_bounds__(THREADS, 1) latent_attention_mma_kernel(const Params p) {
  using T = __nv_bfloat16;
  constexpr int BM = 16 * MT, KG = 8 / MT, TPR = THREADS / BM, CPT = BN / TPR;
  extern __shared__ __align__(128) uint8_t smem[];
  const int DKp = (p.DK + 15) & ~15, kstride = DKp * 2 + 16, chunks = DKp / 8;
  uint8_t *sq = smem, *sk[2] = {sq + BM * kstride, sq + (BM + BN) * kstride};
  float *ss = (float *)(sq + (BM + 2 * BN) * kstride);
  uint8_t *sp = (uint8_t *)(ss + BM * SS);
  float *scorr = (float *)(sp + BM * PB), *sl = scorr + BM;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.y;
  const int tok0 = p.portions ? p.portions[4 * b] : p.cu_tok[b], len = p.portions ? p.portions[4 * b + 1] : p.cu_tok[b + 1] - tok0;
  const int past = p.portions ? p.portions[4 * b + 2] : p.past[b];
  const int32_t *table = p.pages + (int64_t)(p.portions ? p.portions[4 * b + 3] : b) * p.pages_ld;
  const int n_rows = len * p.H, row0 = blockIdx.x * BM;
  if (row0 >= n_rows) return;
  const int tok_lo = row0 / p.H, tok_hi = min(len - 1, (row0 + BM - 1) / p.H);
  const int k_first = p.window > 0 ? max(0, past + tok_lo - p.window + 1) : 0, k_end = past + tok_hi + 1;
  const int nt = (k_end - k_first + BN - 1) / BN;

  auto load_tile = [&](int t, int buf) {
    const int t0 = k_first + t * BN;
    for (int c = tid; c < BN * chunks; c += THREADS) {
      const int row = c / chunks, ch = c % chunks, j = t0 + row;
      const bool ok = j < k_end && ch * 8 < p.DK;
      const int jj = j < k_end ? j : k_first;
      const int64_t at = ((int64_t)table[jj / p.page_size] * p.page_size + jj % p.page_size) * p.cache_row + ch * 8;
      cp_async16(sk[buf] + row * kstride + ch * 16, p.cache + at, ok);
    }
    cp_async_commit();
  };

  for (int c = tid; c < BM * chunks; c += THREADS) {
    const int row = c / chunks, ch = c % chunks, g = row0 + row;
    const bool ok = g < n_rows && ch * 8 < p.DK;
    const int gg = g < n_rows ? g : row0;
    cp_async16(sq + row * kstride + ch * 16, p.q + (int64_t)(tok0 + gg / p.H) * p.q_ld + (int64_t)(gg % p.H) * p.DK + ch * 8, ok);
  }
  cp_async_commit();
  load_tile(0, 0);

  // phase A / C roles
  const int mt = warp % MT, grp = warp / MT;
  const int NT = p.R / 8;                                   // n8 tiles of the output
  int tpg = (NT + KG - 1) / KG;
  tpg = (tpg + 1) & ~1;                                     // whole pairs
  const int tile0 = grp * tpg, my_tiles = max(0, min(NT, tile0 + tpg) - tile0);
  float oacc[MAX_TILES][4];
#pragma unroll
  for (int i = 0; i < MAX_TILES; i++) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f; }
  // phase B role: TPR neighbouring lanes share a row
  const int brow = tid / TPR, bsub = tid % TPR, bg = row0 + brow;
  const int bpos = past + min(bg, n_rows - 1) / p.H;
  float m_run = -INFINITY, l_run = 0.f;

  for (int t = 0; t < nt; t++) {
    const int buf = t & 1;
    cp_async_wait<0>();
    __syncthreads();                       // tile t (and Q) landed; everyone is done with tile t - 1
    if (t + 1 < nt) load_tile(t + 1, buf ^ 1);
    const int t0 = k_first + t * BN;

    {   // ---- A: scores of this warp's rows against its keys
      float sacc[MT][4];
#pragma unroll
      for (int j = 0; j < MT; j++) { sacc[j][0] = sacc[j][1] = sacc[j][2] = sacc[j][3] = 0.f; }
      const int key0 = grp * 8 * MT;
      const uint32_t qa_addr = smem_u32(sq + (mt * 16 + (lane & 15)) * kstride + (lane >> 4) * 16);
#pragma unroll 2
      for (int ks = 0; ks < DKp / 16; ks++) {
        uint32_t a[4];
        ldsm_x4(qa_addr + ks * 32, a[0], a[1], a[2], a[3]);
#pragma unroll
        for (int jp = 0; jp < (MT + 1) / 2; jp++) {
          const int row = key0 + 16 * jp + (lane & 7) + (MT == 1 ? 0 : ((lane >> 4) << 3));
          const int ch = 2 * ks + ((lane >> 3) & 1);
          uint32_t b0, b1, b2, b3;
          ldsm_x4(smem_u32(sk[buf] + row * kstride + ch * 16), b0, b1, b2, b3);
          mma16816<T>(sacc[2 * jp], a, b0, b1);
          if (MT > 1) mma16816<T>(sacc[(2 * jp + 1) % MT], a, b2, b3);
        }
      }
#pragma unroll
      for (int j = 0; j < MT; j++)
#pragma unroll
        for (int e = 0; e < 4; e++)
          ss[(mt * 16 + (lane >> 2) + ((e >> 1) << 3)) * SS + key0 + 8 * j + 2 * (lane & 3) + (e & 1)] = sacc[j][e] * p.scale_log2;
    }
    __syncthreads();

    {   // ---- B: mask, running maximum and sum, P and the rescale factor
      float sv[CPT], mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < CPT; i++) {
        const int col = bsub + i * TPR, key = t0 + col;
        const bool ok = bg < n_rows && key <= bpos && (p.window <= 0 || bpos - key < p.window);
        sv[i] = ok ? ss[brow * SS + col] : -INFINITY;
        mx = fmaxf(mx, sv[i]);
      }
#pragma unroll
      for (int m = 1; m < TPR; m <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, m));
      const float m_new = fmaxf(m_run, mx);
      const float corr = m_new == -INFINITY ? 1.f : exp2f(m_run - m_new);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < CPT; i++) {
        const float pv = m_new == -INFINITY ? 0.f : exp2f(sv[i] - m_new);
        const T pb = __float2bfloat16_rn(pv);
        sum += __bfloat162float(pb);                      // the sum of what the product will use
        *(T *)(sp + brow * PB + (bsub + i * TPR) * 2) = pb;
      }
#pragma unroll
      for (int m = 1; m < TPR; m <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, m);
      l_run = l_run * corr + sum;
      m_run = m_new;
      if (bsub == 0) scorr[brow] = corr;
    }
    __syncthreads();

    {   // ---- C: O = O * corr + P V over this warp's output columns
      const float c0 = scorr[mt * 16 + (lane >> 2)], c1 = scorr[mt * 16 + (lane >> 2) + 8];
#pragma unroll
      for (int i = 0; i < MAX_TILES; i++) { oacc[i][0] *= c0; oacc[i][1] *= c0; oacc[i][2] *= c1; oacc[i][3] *= c1; }
      const uint32_t pa_addr = smem_u32(sp + (mt * 16 + (lane & 15)) * PB + (lane >> 4) * 16);
#pragma unroll
      for (int kk = 0; kk < BN / 16; kk++) {
        uint32_t a[4];
        ldsm_x4(pa_addr + kk * 32, a[0], a[1], a[2], a[3]);
        const int row = 16 * kk + (lane & 7) + (((lane >> 3) & 1) << 3);
#pragma unroll
        for (int dp = 0; dp < MAX_TILES / 2; dp++) {
          if (2 * dp < my_tiles) {
            const int ch = tile0 + 2 * dp + (lane >> 4);
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(smem_u32(sk[buf] + row * kstride + ch * 16), b0, b1, b2, b3);
            mma16816<T>(oacc[2 * dp], a, b0, b1);
            mma16816<T>(oacc[2 * dp + 1], a, b2, b3);
          }
        }
      }
    }
  }
  if (bsub == 0) sl[brow] = l_run;
  __syncthreads();
  const int ra = mt * 16 + (lane >> 2);
  const float l0 = sl[ra], l1 = sl[ra + 8];
  const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
  const int g0 = row0 + ra, g1 = g0 + 8;
  T *o0 = g0 < n_rows ? p.o + (int64_t)(tok0 + g0 / p.H) * p.o_ld + (int64_t)(g0 % p.H) * p.R : nullptr;
  T *o1 = g1 < n_rows ? p.o + (int64_t)(tok0 + g1 / p.H) * p.o_ld + (int64_t)(g1 % p.H) * p.R : nullptr;
#pragma unroll
  for (int i = 0; i < MAX_TILES; i++) {
    if (i < my_tiles) {
      const int col = (tile0 + i) * 8 + 2 * (lane & 3);
      if (o0) *(uint32_t *)(o0 + col) = pack2<T>(oacc[i][0] * inv0, oacc[i][1] * inv0);
      if (o1) *(uint32_t *)(o1 + col) = pack2<T>(oacc[i][2] * inv1, oacc[i][3] * inv1);
    }
  }
}

static size_t smem_bytes(int mt, int dk) {
  const int bm = 16 * mt, dkp = (dk + 15) & ~15, kstride = dkp * 2 + 16;
  return (size_t)(bm + 2 * BN) * kstride + (size_t)bm * SS * 4 + (size_t)bm * PB + (size_t)2 * bm * 4;
}

template <int MT>
static int launch(const Params &p, int n, int longest, cudaStream_t st) {
  auto kern = latent_attention_mma_kernel<MT>;
  const size_t bytes = smem_bytes(MT, p.DK);
  static size_t allowed = 48 * 1024;
  if (bytes > allowed) {
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) return (int)e;
    allowed = bytes;
  }
  kern<<<dim3((longest * p.H + 16 * MT - 1) / (16 * MT), n), THREADS, bytes, st>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace seql

extern "C" int mrs_seq_latent_attention_fits(int kv_rank, int rot_dim) {
  const int dk = kv_rank + rot_dim;
  if (kv_rank < 8 || kv_rank % 8 || dk % 8 || kv_rank > 1024) return 0;
  const int mt = kv_rank <= 256 ? 4 : (kv_rank <= 512 ? 2 : 1);
  return seql::smem_bytes(mt, dk) <= 220 * 1024 ? 1 : 0;
}

extern "C" int mrs_seq_latent_attention(const void *q, int64_t q_ld, const void *cache, int64_t cache_row, void *out, int64_t out_ld,
                                        const int32_t *portions, const int32_t *cu_tok, const int32_t *past, int n_portions, int longest,
                                        const int32_t *pages, int pages_ld, int page_size, int heads, int kv_rank, int rot_dim, float scale,
                                        int window, int64_t stream) {
  if (n_portions <= 0 || longest <= 0) return 0;
  if (heads <= 0 || (!portions && (!cu_tok || !past)) || !pages || page_size <= 0 || !mrs_seq_latent_attention_fits(kv_rank, rot_dim)) return -2;
  if ((q_ld | out_ld | cache_row) % 8 || (((uintptr_t)q | (uintptr_t)cache | (uintptr_t)out) & 15)) return -3;
  seql::Params p = {};
  p.q = (const __nv_bfloat16 *)q; p.cache = (const __nv_bfloat16 *)cache; p.o = (__nv_bfloat16 *)out;
  p.q_ld = q_ld; p.o_ld = out_ld; p.cache_row = cache_row;
  p.portions = portions; p.cu_tok = cu_tok; p.past = past; p.pages = pages; p.pages_ld = pages_ld; p.page_size = page_size;
  p.H = heads; p.DK = kv_rank + rot_dim; p.R = kv_rank;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.window = window;
  cudaStream_t st = (cudaStream_t)stream;
  // row tiles per CTA: as many as the output columns allow, but no more than the longest portion fills (a decoded token's
  // heads are one or two tiles: all eight warps then split its keys and columns)
  const int64_t rows = (int64_t)longest * heads;
  const int by_rank = kv_rank <= 256 ? 4 : (kv_rank <= 512 ? 2 : 1), by_rows = rows <= 16 ? 1 : (rows <= 32 ? 2 : 4);
  const int mt = by_rank < by_rows ? by_rank : by_rows;
  if (mt == 4) return seql::launch<4>(p, n_portions, longest, st);
  if (mt == 2) return seql::launch<2>(p, n_portions, longest, st);
  return seql::launch<1>(p, n_portions, longest, st);
}
