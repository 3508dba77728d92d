// Paged causal attention in bfloat16 on the tensor cores (mma.sync m16n8k16,
// float32 scores, softmax statistics and accumulators), head_dim 64 / 128 / 256,
// any number of heads and groups, any page size.
//
// Rows of a tile are (query token, query head of one kv group) pairs, so the G
// query heads that share a kv head also share every K/V tile that is loaded.
//
//  * attn_decode_kernel: requests with few new tokens (q_len <= max_q_short).  A
//    CTA owns one 16-row tile of one (request, kv head) and ONE SPLIT of its keys;
//    its 4 warps take different 16-key blocks of every 64-key tile and are
//    combined through shared memory at the end.  With more than one split the
//    un-normalised partial results go to scratch; the CTA that finishes a tile last
//    (a counter per tile, reset by that CTA) joins the splits in their fixed order.
//  * attn_prefill_kernel: requests with many new tokens.  A CTA owns 64 rows
//    (4 warps x 16) of one (request, kv head) and walks all visible keys.
//
// Both skip requests that belong to the other kernel, so a mixed step launches
// both.  Cache layer layout: [pages][2 (k, v)][Hkv][page_size][HD].
#include "common.cuh"
#include "tma.cuh"
#include <mutex>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
using namespace bspec;

namespace {

constexpr int KT = 64;          // keys per shared-memory tile
constexpr int NTHREADS = 128;   // 4 warps

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = smem_u32(dst);
  const int n = valid ? 16 : 0;   // src-size 0: the 16 bytes are zero-filled, src is not read
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// element offset of (row, col) in a [rows][HD] bf16 tile whose 16-byte chunks are XOR-swizzled by the row
template <int HD> __device__ __forceinline__ int swz(int row, int col) {
  return row * HD + ((((col >> 3) ^ (row & 7))) << 3) + (col & 7);
}

// the same for a K/V tile written by TMA with its 128-byte swizzle: HD/64 sub-tiles of [KT rows][64 columns]
template <int HD> __device__ __forceinline__ int tswz(int row, int col) {
  return (col >> 6) * (KT * 64) + row * 64 + ((((col & 63) >> 3) ^ (row & 7)) << 3) + (col & 7);
}
template <int HD, bool TMA_TILE> __device__ __forceinline__ int kv_off(int row, int col) {
  return TMA_TILE ? tswz<HD>(row, col) : swz<HD>(row, col);
}

struct TileGeom {
  int e, g, q_begin, q_len, pos0, G, rows_total;
};

// Load K and V rows [k0, k0 + KT) of one kv head into swizzled shared tiles; keys outside [k_lo, k_end) are
// zero-filled and their table entries (which may be released pages) are not read.
template <int HD>
__device__ __forceinline__ void load_kv_tile(__nv_bfloat16* Ks, __nv_bfloat16* Vs, const __nv_bfloat16* cache,
                                             const int* table, int table_page0, int k0, int k_lo, int k_end,
                                             int page_size, int Hkv, int g, long long n_pages) {
  constexpr int CH = HD / 8;                     // 16-byte chunks per row
  const size_t page_elems = (size_t)Hkv * page_size * HD;
  for (int idx = threadIdx.x; idx < KT * CH; idx += NTHREADS) {
    const int row = idx / CH, ch = idx - row * CH;
    const int key = k0 + row;
    bool valid = key < k_end && key >= k_lo;
    const __nv_bfloat16* src = cache;
    if (valid && !bspec::in_range(table[key / page_size - table_page0], n_pages, 108)) valid = false;   // (checked build)
    if (valid) {
      const int pi = key / page_size;
      const int page = table[pi - table_page0];
      src = cache + (size_t)page * 2 * page_elems + ((size_t)g * page_size + (key - pi * page_size)) * HD + ch * 8;
    }
    const int off = row * HD + ((ch ^ (row & 7)) << 3);
    cp_async16(Ks + off, src, valid);
    cp_async16(Vs + off, src + (valid ? page_elems : 0), valid);
  }
}

// Load a 16-row query tile (rows = (token, head in group)) into swizzled shared memory, zero beyond rows_total.
template <int HD>
__device__ __forceinline__ void load_q_tile(__nv_bfloat16* Qs, const __nv_bfloat16* q, long long q_row_stride,
                                            const TileGeom& t, int row0, int nrows) {
  constexpr int CH = HD / 8;
  for (int idx = threadIdx.x; idx < nrows * CH; idx += NTHREADS) {
    const int row = idx / CH, ch = idx - row * CH;
    const int r = row0 + row;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < t.rows_total) {
      const int qi = r / t.G, h = t.g * t.G + (r - qi * t.G);
      v = *reinterpret_cast<const uint4*>(q + (size_t)(t.q_begin + qi) * q_row_stride + (size_t)h * HD + ch * 8);
    }
    *reinterpret_cast<uint4*>(Qs + row * HD + ((ch ^ (row & 7)) << 3)) = v;
  }
}

// One warp: scores of its 16 rows against 16 keys (kb .. kb+15 of the tile), online softmax, P*V.
// qf: A fragments of the rows for every 16-dim step.  Row state (m, l) per thread for rows lane/4 and lane/4+8.
template <int HD, bool TMA_TILE = false>
__device__ __forceinline__ void block16(const uint32_t (&qf)[HD / 16][4], const __nv_bfloat16* Ks,
                                        const __nv_bfloat16* Vs, int kb, int key0, int row_lim0, int row_lim1,
                                        int row_lo0, int row_lo1, int k_end, float scale_log2, float (&m)[2],
                                        float (&l)[2], float (&o)[HD / 8][4]) {
  const int lane = threadIdx.x & 31;
  float s[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
  const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    uint32_t b[4];
    ldmatrix_x4(b, Ks + kv_off<HD, TMA_TILE>(kb + 8 * (mat >> 1) + r8, 16 * ks + 8 * (mat & 1)));
    mma_bf16(s[0], qf[ks], b[0], b[1]);
    mma_bf16(s[1], qf[ks], b[2], b[3]);
  }
  // mask and scale; element i of n-tile nt: row (i >> 1), key column 2*(lane&3) + (i&1)
  float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int key = key0 + kb + 8 * nt + 2 * (lane & 3) + (i & 1);
      const int lim = (i >> 1) ? row_lim1 : row_lim0, lo = (i >> 1) ? row_lo1 : row_lo0;
      const bool ok = key <= lim && key >= lo && key < k_end;
      s[nt][i] = ok ? s[nt][i] * scale_log2 : -INFINITY;
      mx[i >> 1] = fmaxf(mx[i >> 1], s[nt][i]);
    }
  float corr[2], msafe[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float mn = fmaxf(m[r], mx[r]);
    msafe[r] = (mn == -INFINITY) ? 0.f : mn;
    corr[r] = exp2f(m[r] - msafe[r]);          // m = -inf -> 0
    m[r] = mn;
    l[r] *= corr[r];
  }
  uint32_t pf[4];
  {
    float p[2][4];
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        p[nt][i] = exp2f(s[nt][i] - msafe[i >> 1]);
        l[i >> 1] += p[nt][i];
      }
    pf[0] = pack_bf16(p[0][0], p[0][1]);
    pf[1] = pack_bf16(p[0][2], p[0][3]);
    pf[2] = pack_bf16(p[1][0], p[1][1]);
    pf[3] = pack_bf16(p[1][2], p[1][3]);
  }
#pragma unroll
  for (int nd = 0; nd < HD / 8; nd += 2) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[nd][i] *= corr[i >> 1];
      o[nd + 1][i] *= corr[i >> 1];
    }
    uint32_t b[4];
    ldmatrix_x4_trans(b, Vs + kv_off<HD, TMA_TILE>(kb + 8 * (mat & 1) + r8, 8 * (nd + (mat >> 1))));
    mma_bf16(o[nd], pf, b[0], b[1]);
    mma_bf16(o[nd + 1], pf, b[2], b[3]);
  }
}

__device__ __forceinline__ bool tile_geometry(TileGeom& t, const int* qo_indptr, const int* positions, int e, int g,
                                              int Hq, int Hkv) {
  t.e = e;
  t.g = g;
  t.q_begin = qo_indptr[e];
  t.q_len = qo_indptr[e + 1] - t.q_begin;
  if (t.q_len <= 0) return false;
  t.pos0 = positions[t.q_begin];
  t.G = Hq / Hkv;
  t.rows_total = t.q_len * t.G;
  return true;
}

// The end of a split-key CTA, run by its 128 consumer threads: combine the 4 warps through shared memory
// (`scratch_smem`: at least 4*16*HD + 128 floats, no longer used for K/V), write the result (one split) or the
// partial result; with several splits the CTA that gets here last for the tile joins them in split order.
__device__ __forceinline__ void bar_consumers() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <int HD>
__device__ __forceinline__ void decode_finish(float* scratch_smem, int* s_last, float (&m)[2], float (&l)[2],
                                              float (&o)[HD / 8][4], const TileGeom& t, int row0, int g, int e, int rt,
                                              int split, int n_splits, int row_tiles, int Hq, int Hkv,
                                              __nv_bfloat16* __restrict__ out, float* __restrict__ o_part,
                                              float* __restrict__ ml_part, int* __restrict__ tile_counters) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
  // combine the 4 warps through shared memory (reusing the K/V stages)
  float* Os = scratch_smem;                                 // [4][16][HD]
  float* Ms = Os + 4 * 16 * HD;                             // [4][16]
  float* Ls = Ms + 4 * 16;                                  // [4][16]
#pragma unroll
  for (int nd = 0; nd < HD / 8; ++nd)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int row = (lane >> 2) + 8 * (i >> 1), col = 8 * nd + 2 * (lane & 3) + (i & 1);
      Os[(warp * 16 + row) * HD + col] = o[nd][i];
    }
  if ((lane & 3) == 0) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      Ms[warp * 16 + (lane >> 2) + 8 * r] = m[r];
      Ls[warp * 16 + (lane >> 2) + 8 * r] = l[r];
    }
  }
  bar_consumers();
  const int nrows = min(16, t.rows_total - row0);
  for (int idx = threadIdx.x; idx < nrows * HD; idx += NTHREADS) {
    const int row = idx / HD, col = idx - row * HD;
    float mt = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mt = fmaxf(mt, Ms[w * 16 + row]);
    float lt = 0.f, acc = 0.f;
    if (mt != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(Ms[w * 16 + row] - mt);
        lt += Ls[w * 16 + row] * f;
        acc += Os[(w * 16 + row) * HD + col] * f;
      }
    }
    const int r = row0 + row, qi = r / t.G, h = g * t.G + (r - qi * t.G);
    const size_t th = (size_t)(t.q_begin + qi) * Hq + h;
    if (n_splits == 1) {
      out[th * HD + col] = __float2bfloat16_rn(lt > 0.f ? acc / lt : 0.f);
    } else {
      o_part[(th * n_splits + split) * HD + col] = acc;
      if (col == 0) {
        ml_part[(th * n_splits + split) * 2] = mt;
        ml_part[(th * n_splits + split) * 2 + 1] = lt;
      }
    }
  }
  if (n_splits == 1) return;
  // The CTA that gets here last for this tile joins the splits (in split order, so the result does not depend
  // on which CTA it is) and resets the counter for the next launch.
  __threadfence();
  bar_consumers();
  const int tile_id = (e * Hkv + g) * row_tiles + rt;
  if (threadIdx.x == 0) *s_last = (atomicAdd(&tile_counters[tile_id], 1) == n_splits - 1);
  bar_consumers();
  if (!*s_last) return;
  __threadfence();
  float* Wt = Os;                                           // [n_splits <= 64][16] weights exp2(m_s - m)
  float* Inv = Os + 64 * 16;                                // [16]
  for (int row = threadIdx.x; row < nrows; row += NTHREADS) {
    const int r = row0 + row, qi = r / t.G, h = g * t.G + (r - qi * t.G);
    const size_t th = (size_t)(t.q_begin + qi) * Hq + h;
    float mt = -INFINITY;
    for (int sp = 0; sp < n_splits; ++sp) mt = fmaxf(mt, __ldcg(ml_part + (th * n_splits + sp) * 2));
    float lt = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) {
      const float ms = __ldcg(ml_part + (th * n_splits + sp) * 2);
      const float f = (ms == -INFINITY) ? 0.f : exp2f(ms - mt);
      Wt[sp * 16 + row] = f;
      lt += __ldcg(ml_part + (th * n_splits + sp) * 2 + 1) * f;
    }
    Inv[row] = lt > 0.f ? 1.f / lt : 0.f;
  }
  bar_consumers();
  for (int idx = threadIdx.x; idx < nrows * HD; idx += NTHREADS) {
    const int row = idx / HD, col = idx - row * HD;
    const int r = row0 + row, qi = r / t.G, h = g * t.G + (r - qi * t.G);
    const size_t th = (size_t)(t.q_begin + qi) * Hq + h;
    float acc = 0.f;
    for (int sp = 0; sp < n_splits; ++sp) {
      const float f = Wt[sp * 16 + row];
      if (f != 0.f) acc += __ldcg(o_part + (th * n_splits + sp) * HD + col) * f;
    }
    out[th * HD + col] = __float2bfloat16_rn(acc * Inv[row]);
  }
  if (threadIdx.x == 0) tile_counters[tile_id] = 0;
}

// ------------------------------------------------------------------------------------ decode (split keys)
constexpr int TBL_MAX = 1024;   // block-table entries of a split kept in shared memory

template <int HD>
__global__ void __launch_bounds__(NTHREADS)
attn_decode_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride, __nv_bfloat16* __restrict__ out,
                   float* __restrict__ o_part, float* __restrict__ ml_part, int* __restrict__ tile_counters,
                   const __nv_bfloat16* __restrict__ cache, const int* __restrict__ qo_indptr,
                   const int* __restrict__ positions, const int* __restrict__ kv_indptr,
                   const int* __restrict__ kv_indices, int Hq, int Hkv, int page_size, float scale_log2, int window,
                   int n_splits, int row_tiles, int max_q_short, long long n_pages) {
  bspec::pdl_prologue(8);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [16][HD]
  __nv_bfloat16* KV = Qs + 16 * HD;                                        // 2 stages x (K [KT][HD], V [KT][HD])
  int* tbl = reinterpret_cast<int*>(KV + 4 * KT * HD);                     // [TBL_MAX]
  __shared__ int s_last;
  const int split = blockIdx.x, g = blockIdx.y;
  const int e = blockIdx.z / row_tiles, rt = blockIdx.z - e * row_tiles;
  TileGeom t;
  if (!tile_geometry(t, qo_indptr, positions, e, g, Hq, Hkv)) return;
  if (t.q_len > max_q_short) return;
  const int row0 = rt * 16;
  if (row0 >= t.rows_total) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi_lo = row0 / t.G, qi_hi = min(t.q_len - 1, (row0 + 15) / t.G);
  const int hi_key = t.pos0 + qi_hi;
  const int lo_key = window > 0 ? max(0, t.pos0 + qi_lo - window + 1) : 0;
  const int lo_al = (lo_key / KT) * KT;
  const int n_keys = hi_key + 1 - lo_al;
  const int chunk = ((((n_keys + n_splits - 1) / n_splits) + KT - 1) / KT) * KT;
  const int k_begin = lo_al + split * chunk;
  const int k_end = min(hi_key + 1, k_begin + chunk);
  const int* table = kv_indices + kv_indptr[e];
  int table_page0 = 0;

  // per-thread rows: lane/4 and lane/4 + 8 of the tile
  int lim[2], lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + (lane >> 2) + 8 * r;
    const int qi = row / t.G;
    lim[r] = row < t.rows_total ? t.pos0 + qi : -1;
    lo[r] = window > 0 ? max(0, t.pos0 + qi - window + 1) : 0;
  }
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

  if (k_begin < k_end) {
    // the split's block-table entries, once, into shared memory (if they fit)
    const int first_key = max(k_begin, lo_key);
    const int pg0 = first_key / page_size, pg1 = (k_end - 1) / page_size;
    if (pg1 - pg0 + 1 <= TBL_MAX) {
      for (int i = threadIdx.x; i <= pg1 - pg0; i += NTHREADS) tbl[i] = table[pg0 + i];
      table = tbl;
      table_page0 = pg0;
    }
    load_q_tile<HD>(Qs, q, q_row_stride, t, row0, 16);
    __syncthreads();
    const int n_tiles = (k_end - k_begin + KT - 1) / KT;
    load_kv_tile<HD>(KV, KV + KT * HD, cache, table, table_page0, k_begin, lo_key, k_end, page_size, Hkv, g, n_pages);
    cp_async_commit();
    uint32_t qf[HD / 16][4];
    {
      const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks], Qs + swz<HD>(8 * (mat & 1) + r8, 16 * ks + 8 * (mat >> 1)));
    }
    for (int it = 0; it < n_tiles; ++it) {
      __nv_bfloat16* Ks = KV + (it & 1) * 2 * KT * HD;
      __nv_bfloat16* Vs = Ks + KT * HD;
      if (it + 1 < n_tiles) {
        __nv_bfloat16* Kn = KV + ((it + 1) & 1) * 2 * KT * HD;
        load_kv_tile<HD>(Kn, Kn + KT * HD, cache, table, table_page0, k_begin + (it + 1) * KT, lo_key, k_end,
                         page_size, Hkv, g, n_pages);
        cp_async_commit();
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const int key0 = k_begin + it * KT;
      if (key0 + 16 * warp < k_end)
        block16<HD>(qf, Ks, Vs, 16 * warp, key0, lim[0], lim[1], lo[0], lo[1], k_end, scale_log2, m, l, o);
      __syncthreads();
    }
  }
  decode_finish<HD>(reinterpret_cast<float*>(KV), &s_last, m, l, o, t, row0, g, e, rt, split, n_splits, row_tiles, Hq,
                    Hkv, out, o_part, ml_part, tile_counters);
}

// ------------------------------------------------------------------------------------ decode, K/V through TMA
// The same split-key work as attn_decode_kernel, for page sizes 8 / 16 / 32 / 64: a fifth warp feeds a ring of
// K/V stages with TMA tensor copies (one box per page and 64-column half, 128-byte swizzle, completion on an
// mbarrier), so the four consumer warps spend no instructions on addresses.  A tile always loads whole pages;
// pages outside the split's range are replaced by its nearest needed page (their keys are masked anyway), so
// shared memory never holds bytes that were not read from the cache.  The cache must not hold NaN or infinity in
// rows that were never written (the pool is allocated zeroed).
constexpr int TMA_STAGES = 3;
constexpr int DECODE_TMA_THREADS = 160;

template <int HD>
__global__ void __launch_bounds__(DECODE_TMA_THREADS)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* __restrict__ q,
                       long long q_row_stride, __nv_bfloat16* __restrict__ out, float* __restrict__ o_part,
                       float* __restrict__ ml_part, int* __restrict__ tile_counters, int* __restrict__ status,
                       const int* __restrict__ qo_indptr, const int* __restrict__ positions,
                       const int* __restrict__ kv_indptr, const int* __restrict__ kv_indices, int Hq, int Hkv,
                       int page_size, float scale_log2, int window, int n_splits, int row_tiles, int max_q_short) {
  // The step's metadata (lengths, positions, block tables) was uploaded before the step's first kernel, and every
  // cached key below the first new token was written by earlier steps: the producer may fetch those tiles while
  // the kernel before this one (which writes q and the new tokens' keys and values) is still running.
  const unsigned long long t_trace = bspec::g_trace_buf != nullptr ? bspec::global_timer() : 0ull;
  bspec::pdl_launch_dependents();
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  constexpr int TILE_ELEMS = KT * HD;                                        // one K (or V) tile
  __nv_bfloat16* KV = reinterpret_cast<__nv_bfloat16*>(smem);                // TMA_STAGES x (K tile, V tile)
  __nv_bfloat16* Qs = KV + TMA_STAGES * 2 * TILE_ELEMS;                      // [16][HD]
  uint64_t* full = reinterpret_cast<uint64_t*>(Qs + 16 * HD);
  uint64_t* empty = full + TMA_STAGES;
  int* tbl = reinterpret_cast<int*>(empty + TMA_STAGES);                     // [TBL_MAX]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tbl + TBL_MAX);
  int* s_last = const_cast<int*>(abort_flag) + 1;

  const int split = blockIdx.x, g = blockIdx.y;
  const int e = blockIdx.z / row_tiles, rt = blockIdx.z - e * row_tiles;
  TileGeom t;
  if (!tile_geometry(t, qo_indptr, positions, e, g, Hq, Hkv)) return;
  if (t.q_len > max_q_short) return;
  const int row0 = rt * 16;
  if (row0 >= t.rows_total) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi_lo = row0 / t.G, qi_hi = min(t.q_len - 1, (row0 + 15) / t.G);
  const int hi_key = t.pos0 + qi_hi;
  const int lo_key = window > 0 ? max(0, t.pos0 + qi_lo - window + 1) : 0;
  const int lo_al = (lo_key / KT) * KT;
  const int n_keys = hi_key + 1 - lo_al;
  const int chunk = ((((n_keys + n_splits - 1) / n_splits) + KT - 1) / KT) * KT;
  const int k_begin = lo_al + split * chunk;
  const int k_end = min(hi_key + 1, k_begin + chunk);
  const int n_tiles = k_begin < k_end ? (k_end - k_begin + KT - 1) / KT : 0;
  const int* table = kv_indices + kv_indptr[e];

  if (threadIdx.x == 0) {
    for (int s = 0; s < TMA_STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 4);          // one arrival per consumer warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

  if (warp == 4) {
    // ---- producer: the copies of a key tile are dealt to the lanes (see attn_decode_shares_kernel)
    if (n_tiles > 0) {
      const int first_pg = max(k_begin, lo_key) / page_size, last_pg = (k_end - 1) / page_size;
      const int n_pg = last_pg - first_pg + 1;
      const bool in_smem = n_pg <= TBL_MAX;
      if (in_smem) {
        for (int i = lane; i < n_pg; i += 32) tbl[i] = table[first_pg + i];
        __syncwarp();
      }
      const int pages_per_tile = KT / page_size;
      constexpr uint32_t tile_bytes = 2u * TILE_ELEMS * 2u;
      constexpr int PER_PAGE = 2 * (HD / 64);
      bool waited = false;
      int ok = 1;
      for (int it = 0; it < n_tiles; ++it) {
        const int s = it % TMA_STAGES;
        const uint32_t ph = (uint32_t)(it / TMA_STAGES) & 1u;
        if (!waited && (it >= TMA_STAGES || k_begin + (it + 1) * KT > t.pos0)) {
          bspec::pdl_wait();             // this tile holds new keys, or a stage must first be released by consumers
          waited = true;
        }
        if (lane == 0) {
          ok = mbar_wait(empty + s, ph ^ 1u, abort_flag, status, 11) ? 1 : 0;
          if (ok) mbar_expect_tx(full + s, tile_bytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        __nv_bfloat16* Ks = KV + (size_t)s * 2 * TILE_ELEMS;
        const int key0 = k_begin + it * KT;
        for (int bx = lane; bx < pages_per_tile * PER_PAGE; bx += 32) {
          const int pp = bx / PER_PAGE, rem = bx - pp * PER_PAGE, c = rem >> 1, is_v = rem & 1;
          int pg = key0 / page_size + pp;
          pg = min(max(pg, first_pg), last_pg);
          const int page = in_smem ? tbl[pg - first_pg] : table[pg];
          const int row = ((page * 2 + is_v) * Hkv + g) * page_size;           // first cache row of this page's K (or V)
          tma_load_2d(Ks + is_v * TILE_ELEMS + c * (KT * 64) + pp * page_size * 64, &kv_map, full + s, c * 64, row);
        }
      }
    }
    return;
  }

  // ---- consumers (threads 0..127)
  bspec::pdl_wait();
  bspec::trace_record(8, t_trace);
  int lim[2], lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + (lane >> 2) + 8 * r;
    const int qi = row / t.G;
    lim[r] = row < t.rows_total ? t.pos0 + qi : -1;
    lo[r] = window > 0 ? max(0, t.pos0 + qi - window + 1) : 0;
  }
  if (n_tiles > 0) {
    load_q_tile<HD>(Qs, q, q_row_stride, t, row0, 16);
    bar_consumers();
    uint32_t qf[HD / 16][4];
    {
      const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks)
        ldmatrix_x4(qf[ks], Qs + swz<HD>(8 * (mat & 1) + r8, 16 * ks + 8 * (mat >> 1)));
    }
    for (int it = 0; it < n_tiles; ++it) {
      const int s = it % TMA_STAGES;
      const uint32_t ph = (uint32_t)(it / TMA_STAGES) & 1u;
      if (!mbar_wait(full + s, ph, abort_flag, status, 12)) break;
      const __nv_bfloat16* Ks = KV + (size_t)s * 2 * TILE_ELEMS;
      const int key0 = k_begin + it * KT;
      if (key0 + 16 * warp < k_end)
        block16<HD, true>(qf, Ks, Ks + TILE_ELEMS, 16 * warp, key0, lim[0], lim[1], lo[0], lo[1], k_end, scale_log2,
                          m, l, o);
      __syncwarp();
      if (lane == 0) mbar_arrive(empty + s);
    }
  }
  bar_consumers();                        // every warp is done with the stages (or gave up)
  if (*abort_flag) return;
  decode_finish<HD>(reinterpret_cast<float*>(KV), s_last, m, l, o, t, row0, g, e, rt, split, n_splits, row_tiles, Hq,
                    Hkv, out, o_part, ml_part, tile_counters);
}

template <int HD> size_t decode_tma_smem() {
  return 1024 + (size_t)TMA_STAGES * 2 * KT * HD * 2 + (size_t)16 * HD * 2 + 2 * TMA_STAGES * 8 + (size_t)TBL_MAX * 4 + 64;
}

// ------------------------------------------------------------------------------------ decode, equal shares
// The same work as attn_decode_tma_kernel, cut differently.  All 64-key tiles of the launch form one sequence
// (request by request, kv head by kv head, row tile by row tile, keys in order), and CTA b of R takes the tiles
// [b T / R, (b + 1) T / R): every CTA streams the same number of tiles however different the requests' lengths are,
// and its producer warp fetches the next piece's keys while the consumers still finish the last one.  A (request,
// kv head, row tile) that lies inside one CTA's share is written at once; one that is spread over several CTAs
// leaves one partial result per CTA, and the CTA that announces the last of them (a counter per row tile, reset
// by that CTA) joins them in their order.  The cut depends only on the lengths of this launch's requests, so a
// captured launch follows each replay's lengths.
constexpr int BAL_MAX_ENTRIES = 512;   // requests of a launch (their tile counts are scanned in shared memory)
constexpr int BAL_TBL = 512;           // block-table entries of a piece kept in shared memory
constexpr int BAL_MIN_SHARE = 2;       // tiles: fewer CTAs take part rather than shares below this

// What all CTAs (and the join) agree on: tiles before each request, the tiles in all, the CTAs that take part.
struct Shares {
  const int* cum;        // [n_entries + 1], tiles of a request = (cum[e + 1] - cum[e]) for ALL its kv heads and row tiles
  long long total;
  int ctas;
  __device__ __forceinline__ long long start_of(int b) const { return (long long)b * total / ctas; }
  __device__ __forceinline__ int cta_of(long long p) const { return (int)(((p + 1) * ctas - 1) / total); }
};

struct Piece {
  TileGeom t;
  int e, g, rt, row0, k_begin, k_end, n_tiles, lo_key;
  int part, n_parts;     // which partial result of the row tile this is, of how many (1: written at once)
  int tiles_taken;       // tiles of the sequence this piece covers (>= n_tiles: masked tiles are not fetched)
};

// The piece that starts at position `pos` of the sequence and ends with its row tile or with the CTA's share.
__device__ __forceinline__ void piece_at(Piece& pc, long long pos, long long share_end, int b, const Shares& sh,
                                         const int* pos0_of, const int* rows_of, int n_entries, int Hq, int Hkv,
                                         int row_tiles, int window) {
  int lo = 0, hi = n_entries;                    // largest e with cum[e] <= pos
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (sh.cum[mid] <= pos) lo = mid; else hi = mid;
  }
  const int e = lo;
  const int tiles_e = (sh.cum[e + 1] - sh.cum[e]) / (Hkv * row_tiles);
  const int rel = (int)(pos - sh.cum[e]);
  const int pair = rel / tiles_e, t0 = rel - pair * tiles_e;
  const int t1 = (int)min((long long)tiles_e, t0 + (share_end - pos));
  pc.tiles_taken = t1 - t0;
  pc.e = e;
  pc.g = pair / row_tiles;
  pc.rt = pair - pc.g * row_tiles;
  const long long pair_start = sh.cum[e] + (long long)pair * tiles_e;
  const int first = sh.cta_of(pair_start);
  pc.n_parts = sh.cta_of(pair_start + tiles_e - 1) - first + 1;
  pc.part = b - first;
  TileGeom& t = pc.t;
  t.e = e;
  t.g = pc.g;
  t.q_begin = rows_of[e] & ((1 << 26) - 1);
  t.q_len = rows_of[e] >> 26;
  t.pos0 = pos0_of[e];
  t.G = Hq / Hkv;
  t.rows_total = t.q_len * t.G;
  pc.row0 = pc.rt * 16;
  pc.n_tiles = 0;
  pc.k_begin = pc.k_end = pc.lo_key = 0;
  if (pc.row0 >= t.rows_total) return;
  const int qi_lo = pc.row0 / t.G, qi_hi = min(t.q_len - 1, (pc.row0 + 15) / t.G);
  const int hi_key = t.pos0 + qi_hi;
  pc.lo_key = window > 0 ? max(0, t.pos0 + qi_lo - window + 1) : 0;
  const int lo_entry = window > 0 ? max(0, t.pos0 - window + 1) : 0;      // the request's tiles start here
  const int lo_al = (lo_entry / KT) * KT;
  pc.k_begin = lo_al + t0 * KT;
  pc.k_end = min(hi_key + 1, lo_al + t1 * KT);
  if (pc.k_begin < pc.k_end && pc.lo_key < pc.k_end) pc.n_tiles = (pc.k_end - pc.k_begin + KT - 1) / KT;
}

// Tiles per request and their running sum (all threads of the CTA call this); also every request's first position
// (pos0_of) and its first row with its number of new tokens (rows_of: q_begin | q_len << 26; q_len <= 16).
// Returns false if the launch has no tiles at all.
__device__ __forceinline__ bool make_shares(Shares& sh, int* cum, int* pos0_of, int* rows_of, int* red, int n_entries,
                                            const int* __restrict__ qo_indptr, const int* __restrict__ positions,
                                            const int* __restrict__ kv_len, int Hkv, int row_tiles, int window,
                                            int max_parts, int max_q_short, int n_threads, int grid) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int most = 0, fewest = 0x7fffffff, live = 0;
  for (int e = threadIdx.x; e < n_entries; e += n_threads) {
    const int qb = qo_indptr[e], ql = qo_indptr[e + 1] - qb;
    const int len_after = kv_len != nullptr ? kv_len[e] : 0;     // asked for together with the two loads above
    int tiles = 0, pos0 = 0;
    if (ql > 0 && ql <= max_q_short) {
      pos0 = kv_len != nullptr ? len_after - ql : positions[qb];
      const int lo_entry = window > 0 ? max(0, pos0 - window + 1) : 0;
      tiles = (pos0 + ql - (lo_entry / KT) * KT + KT - 1) / KT;
    }
    pos0_of[e] = pos0;
    rows_of[e] = qb | (tiles > 0 ? ql << 26 : 0);
    cum[e + 1] = tiles * Hkv * row_tiles;
    most = max(most, tiles);
    if (tiles > 0) {
      fewest = min(fewest, tiles);
      ++live;
    }
  }
  if (threadIdx.x == 0) { cum[0] = 0; red[0] = 0; red[1] = 0x7fffffff; red[2] = 0; }
  __syncthreads();
  atomicMax(&red[0], most);
  atomicMin(&red[1], fewest);
  if (live) atomicAdd(&red[2], live);
  if (warp == 0) {                       // inclusive scan, 32 requests at a time
    int carry = 0;
    for (int base = 0; base < n_entries; base += 32) {
      int v = base + lane < n_entries ? cum[base + lane + 1] : 0;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += y;
      }
      if (base + lane < n_entries) cum[base + lane + 1] = v + carry;
      carry += __shfl_sync(0xffffffffu, v, 31);
    }
  }
  __syncthreads();
  sh.cum = cum;
  sh.total = cum[n_entries];
  if (sh.total <= 0) return false;
  // a row tile of `most` tiles must not be spread over more than max_parts shares
  const int least = max(BAL_MIN_SHARE, (red[0] + max_parts - 3) / (max_parts - 2));
  sh.ctas = (int)max(1ll, min((long long)grid, sh.total / least));
  // Requests of one length, and fewer row tiles than CTAs: give every row tile the same whole number of CTAs, so
  // that no share reaches into the next row tile (a second piece costs a CTA about as much as four tiles).
  const long long pairs = (long long)red[2] * Hkv * row_tiles;
  if (red[0] == red[1] && pairs <= sh.ctas) {
    const int per_pair = (int)min((long long)sh.ctas / pairs, (long long)max(1, red[0] / least));
    const long long aligned = pairs * per_pair;
    // tiles a CTA streams either way; a share that reaches into a second row tile pays for about four more
    if (sh.total / aligned <= sh.total / sh.ctas + 4) sh.ctas = (int)aligned;
  }
  return true;
}

// Joins the n_parts partial results of one row tile (in their order, so the result does not depend on which CTA
// does it).  Called by the 128 consumer threads; Wt: 64 * 16 + 16 floats of shared memory.
template <int HD>
__device__ __forceinline__ void join_parts(float* Wt, __nv_bfloat16* __restrict__ out, const float* __restrict__ o_part,
                                           const float* __restrict__ ml_part, int e, int g, int row0, int q_begin,
                                           int rows_total, int G, int Hq, int n_parts, int max_parts, int rows_pe) {
  const int nrows = min(16, rows_total - row0);
  float* Inv = Wt + 64 * 16;
  {
    // weights of the partial results: 8 threads per row, each with the parts sp = j, j + 8, ... (at most 8 of 64)
    const int row = threadIdx.x >> 3, j8 = threadIdx.x & 7;
    const bool live = row < nrows;
    const int r = row0 + (live ? row : 0), qi = r / G, h = g * G + (r - qi * G);
    const size_t ph = (size_t)(e * rows_pe + qi) * Hq + h;
    float ms[8], ls[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int sp = j8 + 8 * u;
      const bool in = live && sp < n_parts;
      ms[u] = in ? __ldcg(ml_part + (ph * max_parts + sp) * 2) : -INFINITY;
      ls[u] = in ? __ldcg(ml_part + (ph * max_parts + sp) * 2 + 1) : 0.f;
    }
    float mt = -INFINITY;
#pragma unroll
    for (int u = 0; u < 8; ++u) mt = fmaxf(mt, ms[u]);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
    float lt = 0.f;
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int sp = j8 + 8 * u;
      const float f = (ms[u] == -INFINITY) ? 0.f : exp2f(ms[u] - mt);
      if (live && sp < n_parts) Wt[sp * 16 + row] = f;
      lt += ls[u] * f;
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) lt += __shfl_xor_sync(0xffffffffu, lt, o);
    if (live && j8 == 0) Inv[row] = lt > 0.f ? 1.f / lt : 0.f;
  }
  bar_consumers();
  for (int idx = threadIdx.x; idx < nrows * (HD / 4); idx += NTHREADS) {
    const int row = idx / (HD / 4), c4 = idx - row * (HD / 4);
    const int r = row0 + row, qi = r / G, h = g * G + (r - qi * G);
    const float* src = o_part + ((size_t)(e * rows_pe + qi) * Hq + h) * max_parts * HD + 4 * c4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    int sp = 0;
    for (; sp + 4 <= n_parts; sp += 4) {                  // four loads in flight; the order of the sum is fixed
      float4 v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) v[u] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + u) * HD));
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float f = Wt[(sp + u) * 16 + row];
        acc.x += v[u].x * f; acc.y += v[u].y * f; acc.z += v[u].z * f; acc.w += v[u].w * f;
      }
    }
    for (; sp < n_parts; ++sp) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * HD));
      const float f = Wt[sp * 16 + row];
      acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
    }
    const float inv = Inv[row];
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(out + ((size_t)(q_begin + qi) * Hq + h) * HD + 4 * c4) = packed;
  }
  bar_consumers();
}

template <int HD>
__global__ void __launch_bounds__(DECODE_TMA_THREADS)
attn_decode_shares_kernel(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* __restrict__ q,
                          long long q_row_stride, __nv_bfloat16* __restrict__ out, float* __restrict__ o_part,
                          float* __restrict__ ml_part, int* __restrict__ tile_counters, int* __restrict__ status,
                          const int* __restrict__ qo_indptr, const int* __restrict__ positions,
                          const int* __restrict__ kv_len,
                          const int* __restrict__ kv_indptr, const int* __restrict__ kv_indices, int n_entries, int Hq,
                          int Hkv, int page_size, float scale_log2, int window, int max_parts, int rows_pe,
                          int row_tiles, int max_q_short) {
  // Lengths, positions and block tables were uploaded before the step's first kernel, and every cached key below
  // the first new token was written by earlier steps: all of that may be read, and those tiles fetched, while the
  // kernel before this one (which writes q and the new tokens' keys and values) still runs.
  const unsigned long long t_trace = bspec::g_trace_buf != nullptr ? bspec::global_timer() : 0ull;
  bspec::pdl_launch_dependents();
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  constexpr int TILE_ELEMS = KT * HD;
  __nv_bfloat16* KV = reinterpret_cast<__nv_bfloat16*>(smem);                // TMA_STAGES x (K tile, V tile)
  __nv_bfloat16* Qs = KV + TMA_STAGES * 2 * TILE_ELEMS;                      // [16][HD]
  uint64_t* full = reinterpret_cast<uint64_t*>(Qs + 16 * HD);
  uint64_t* empty = full + TMA_STAGES;
  float* MsLs = reinterpret_cast<float*>(empty + TMA_STAGES);                // [224] the combine's small arrays
  int* cum = reinterpret_cast<int*>(MsLs + 224);                             // [BAL_MAX_ENTRIES + 1]
  int* pos0_of = cum + BAL_MAX_ENTRIES + 1;                                  // [BAL_MAX_ENTRIES]
  int* rows_of = pos0_of + BAL_MAX_ENTRIES;                                  // [BAL_MAX_ENTRIES]
  int* tbl = rows_of + BAL_MAX_ENTRIES;                                      // [BAL_TBL]
  int* red = tbl + BAL_TBL;                                                  // [3]
  volatile int* abort_flag = reinterpret_cast<volatile int*>(red + 3);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < TMA_STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 4);          // one arrival per consumer warp
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  Shares sh;
  if (!make_shares(sh, cum, pos0_of, rows_of, red, n_entries, qo_indptr, positions, kv_len, Hkv, row_tiles, window, max_parts,
                   max_q_short, DECODE_TMA_THREADS, gridDim.x))
    return;
  const int b = blockIdx.x;
  if (b >= sh.ctas) return;
  const long long share_begin = sh.start_of(b), share_end = sh.start_of(b + 1);
  uint32_t tile_no = 0;                  // tiles this CTA has been through: stage and phase follow from it

  if (warp == 4) {
    // ---- producer: the copies of a key tile are dealt to the lanes (a single thread issuing all sixteen 2 KB
    // copies of a tile runs at about two thirds of what one thread can issue at all)
    bool waited = false;
    int ok = 1;
    const int pages_per_tile = KT / page_size;
    for (long long pos = share_begin; pos < share_end && ok;) {
      Piece pc;
      piece_at(pc, pos, share_end, b, sh, pos0_of, rows_of, n_entries, Hq, Hkv, row_tiles, window);
      pos += pc.tiles_taken;
      if (pc.n_tiles == 0) continue;
      const int* table = kv_indices + kv_indptr[pc.e];
      const int first_pg = max(pc.k_begin, pc.lo_key) / page_size, last_pg = (pc.k_end - 1) / page_size;
      const int n_pg = last_pg - first_pg + 1;
      const bool in_smem = n_pg <= BAL_TBL;
      __syncwarp();
      if (in_smem)
        for (int i = lane; i < n_pg; i += 32) tbl[i] = table[first_pg + i];
      __syncwarp();
      constexpr uint32_t tile_bytes = 2u * TILE_ELEMS * 2u;
      for (int k = 0; k < pc.n_tiles; ++k, ++tile_no) {
        const int s = tile_no % TMA_STAGES;
        const uint32_t ph = (tile_no / TMA_STAGES) & 1u;
        if (!waited && (tile_no >= TMA_STAGES || pc.k_begin + (k + 1) * KT > pc.t.pos0)) {
          bspec::pdl_wait();           // this tile holds new keys, or a stage must first be released by consumers
          waited = true;
        }
        if (lane == 0) {
          ok = mbar_wait(empty + s, ph ^ 1u, abort_flag, status, 13) ? 1 : 0;
          if (ok) mbar_expect_tx(full + s, tile_bytes);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        // the tile's copies, one per (page, 64-column half, K or V), dealt to the lanes
        __nv_bfloat16* Ks = KV + (size_t)s * 2 * TILE_ELEMS;
        constexpr int PER_PAGE = 2 * (HD / 64);
        for (int bx = lane; bx < pages_per_tile * PER_PAGE; bx += 32) {
          const int pp = bx / PER_PAGE, rem = bx - pp * PER_PAGE, c = rem >> 1, is_v = rem & 1;
          int pg = (pc.k_begin + k * KT) / page_size + pp;
          pg = min(max(pg, first_pg), last_pg);
          const int page = in_smem ? tbl[pg - first_pg] : table[pg];
          const int row = ((page * 2 + is_v) * Hkv + pc.g) * page_size;       // first cache row of this page's K (or V)
          tma_load_2d(Ks + is_v * TILE_ELEMS + c * (KT * 64) + pp * page_size * 64, &kv_map, full + s, c * 64, row);
        }
      }
    }
    return;
  }

  // ---- consumers (threads 0..127)
  bspec::pdl_wait();
  bspec::trace_record(8, t_trace);
  // Only the first and the last row tile of a share can be shared with other CTAs: their partial results are
  // announced after all of the share's streaming, so that the wait for those writes to land is paid once.
  int n_pending = 0, pend_e[2], pend_g[2], pend_rt[2], pend_parts[2];
  bool aborted = false;
  for (long long pos = share_begin; pos < share_end;) {
    Piece pc;
    piece_at(pc, pos, share_end, b, sh, pos0_of, rows_of, n_entries, Hq, Hkv, row_tiles, window);
    pos += pc.tiles_taken;
    if (pc.row0 >= pc.t.rows_total) continue;               // no such row tile in this request: nothing to write
    const TileGeom& t = pc.t;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o[i][j] = 0.f;
    int last_stage = -1;
    if (pc.n_tiles > 0) {
      int lim[2], lo[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int row = pc.row0 + (lane >> 2) + 8 * r;
        const int qi = row / t.G;
        lim[r] = row < t.rows_total ? t.pos0 + qi : -1;
        lo[r] = window > 0 ? max(0, t.pos0 + qi - window + 1) : 0;
      }
      load_q_tile<HD>(Qs, q, q_row_stride, t, pc.row0, 16);
      bar_consumers();
      uint32_t qf[HD / 16][4];
      {
        const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks)
          ldmatrix_x4(qf[ks], Qs + swz<HD>(8 * (mat & 1) + r8, 16 * ks + 8 * (mat >> 1)));
      }
      for (int k = 0; k < pc.n_tiles; ++k, ++tile_no) {
        const int s = tile_no % TMA_STAGES;
        const uint32_t ph = (tile_no / TMA_STAGES) & 1u;
        if (!mbar_wait(full + s, ph, abort_flag, status, 14)) break;   // the flag is set: all warps leave below
        const __nv_bfloat16* Ks = KV + (size_t)s * 2 * TILE_ELEMS;
        const int key0 = pc.k_begin + k * KT;
        if (key0 + 16 * warp < pc.k_end)
          block16<HD, true>(qf, Ks, Ks + TILE_ELEMS, 16 * warp, key0, lim[0], lim[1], lo[0], lo[1], pc.k_end,
                            scale_log2, m, l, o);
        __syncwarp();
        if (k + 1 < pc.n_tiles) {
          if (lane == 0) mbar_arrive(empty + s);
        } else {
          last_stage = s;                                   // kept for the combine below
        }
      }
    }
    bar_consumers();                     // every warp is done with the last tile's keys (and with Qs)
    if (*abort_flag) { aborted = true; break; }
    if (pc.n_parts > 1 && n_pending < 2) {
      pend_e[n_pending] = pc.e; pend_g[n_pending] = pc.g; pend_rt[n_pending] = pc.rt; pend_parts[n_pending] = pc.n_parts;
      ++n_pending;
    }

    // ---- combine the 4 warps (in the last tile's stage), write the result or the partial result
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
      l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    // Os: [4 warps][16 rows][HD] with the 4-float groups of a row XOR-ed by the row (no bank conflicts either way)
    float* Os = last_stage >= 0 ? reinterpret_cast<float*>(KV + (size_t)last_stage * 2 * TILE_ELEMS) : nullptr;
    float* Ms = MsLs;
    float* Ls = MsLs + 64;
    float* Fs = MsLs + 128;              // [4][16] weight of each warp's share of a row; [16] the row's sum after it
    if (Os != nullptr) {
#pragma unroll
      for (int nd = 0; nd < HD / 8; ++nd)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int row = (lane >> 2) + 8 * r, col = 8 * nd + 2 * (lane & 3);
          *reinterpret_cast<float2*>(Os + (warp * 16 + row) * HD + ((((col >> 2) ^ (row & 7)) << 2) | (col & 3))) =
              make_float2(o[nd][2 * r], o[nd][2 * r + 1]);
        }
      if ((lane & 3) == 0) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          Ms[warp * 16 + (lane >> 2) + 8 * r] = m[r];
          Ls[warp * 16 + (lane >> 2) + 8 * r] = l[r];
        }
      }
    }
    bar_consumers();
    if (threadIdx.x < 16) {
      const int row = threadIdx.x;
      float mt = -INFINITY, lt = 0.f;
      if (Os != nullptr) {
#pragma unroll
        for (int w = 0; w < 4; ++w) mt = fmaxf(mt, Ms[w * 16 + row]);
      }
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = mt == -INFINITY ? 0.f : exp2f(Ms[w * 16 + row] - mt);
        Fs[w * 16 + row] = f;
        lt += mt == -INFINITY ? 0.f : Ls[w * 16 + row] * f;
      }
      Fs[64 + row] = lt;
      Fs[80 + row] = mt;
    }
    bar_consumers();
    const int nrows = min(16, t.rows_total - pc.row0);
    for (int idx = threadIdx.x; idx < nrows * (HD / 4); idx += NTHREADS) {
      const int row = idx / (HD / 4), c4 = idx - row * (HD / 4);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (Os != nullptr) {
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float f = Fs[w * 16 + row];
          const float4 v = *reinterpret_cast<const float4*>(Os + (w * 16 + row) * HD + ((c4 ^ (row & 7)) << 2));
          acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
      }
      const float lt = Fs[64 + row];
      const int r = pc.row0 + row, qi = r / t.G, h = pc.g * t.G + (r - qi * t.G);
      if (pc.n_parts == 1) {
        const float inv = lt > 0.f ? 1.f / lt : 0.f;
        uint2 packed;
        packed.x = pack_bf16(acc.x * inv, acc.y * inv);
        packed.y = pack_bf16(acc.z * inv, acc.w * inv);
        *reinterpret_cast<uint2*>(out + ((size_t)(t.q_begin + qi) * Hq + h) * HD + 4 * c4) = packed;
      } else {
        const size_t ph = (size_t)(pc.e * rows_pe + qi) * Hq + h;     // partial results: by request and its row
        *reinterpret_cast<float4*>(o_part + (ph * max_parts + pc.part) * HD + 4 * c4) = acc;
        if (c4 == 0) {
          ml_part[(ph * max_parts + pc.part) * 2] = Fs[80 + row];
          ml_part[(ph * max_parts + pc.part) * 2 + 1] = lt;
        }
      }
    }
    // hand the stage back: the copies that will overwrite it run in the asynchronous proxy
    if (last_stage >= 0) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      bar_consumers();
      if (lane == 0) mbar_arrive(empty + last_stage);
    }
  }
  if (aborted || n_pending == 0) return;
  // The CTA that announces a row tile's last partial result joins them and resets the counter for the next launch.
  __threadfence();
  bar_consumers();
  if ((int)threadIdx.x < n_pending) {
    const int i = threadIdx.x;
    const int tile_id = (pend_e[i] * Hkv + pend_g[i]) * row_tiles + pend_rt[i];
    red[i] = atomicAdd(&tile_counters[tile_id], 1) == pend_parts[i] - 1;
    if (red[i]) tile_counters[tile_id] = 0;
  }
  bar_consumers();
  float* Wt = reinterpret_cast<float*>(KV);     // every tile of this CTA has been consumed: the stages are free
  for (int i = 0; i < n_pending; ++i) {
    if (!red[i]) continue;
    __threadfence();
    const int e = pend_e[i], q_begin = rows_of[e] & ((1 << 26) - 1), q_len = rows_of[e] >> 26, G = Hq / Hkv;
    join_parts<HD>(Wt, out, o_part, ml_part, e, pend_g[i], pend_rt[i] * 16, q_begin, q_len * G, G, Hq, pend_parts[i],
                   max_parts, rows_pe);
  }
}

template <int HD> size_t decode_shares_smem() {
  return 1024 + (size_t)TMA_STAGES * 2 * KT * HD * 2 + (size_t)16 * HD * 2 + 2 * TMA_STAGES * 8 + (size_t)224 * 4 +
         (size_t)(3 * BAL_MAX_ENTRIES + 1 + BAL_TBL + 4) * 4 + 64;
}

// ------------------------------------------------------------------------------------ prefill, 128 rows, TMA
// One warp: scores of its 16 rows against all 64 keys of a tile, one online-softmax step, P*V.
template <int HD, bool TMA_TILE>
__device__ __forceinline__ void block64(const uint32_t (&qf)[HD / 16][4], const __nv_bfloat16* Ks,
                                        const __nv_bfloat16* Vs, int key0, int row_lim0, int row_lim1, int row_lo0,
                                        int row_lo1, int k_end, bool need_mask, float scale_log2, float (&m)[2],
                                        float (&l)[2], float (&o)[HD / 8][4]) {
  const int lane = threadIdx.x & 31;
  const int mat = lane >> 3, r8 = lane & 7;
  float s[8][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt)
#pragma unroll
    for (int i = 0; i < 4; ++i) s[nt][i] = 0.f;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      uint32_t b[4];
      ldmatrix_x4(b, Ks + kv_off<HD, TMA_TILE>(16 * np + 8 * (mat >> 1) + r8, 16 * ks + 8 * (mat & 1)));
      mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
      mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
    }
  }
  float mx[2] = {-INFINITY, -INFINITY};
  if (need_mask) {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = key0 + 8 * nt + 2 * (lane & 3) + (i & 1);
        const int lim = (i >> 1) ? row_lim1 : row_lim0, lo = (i >> 1) ? row_lo1 : row_lo0;
        const bool ok = key <= lim && key >= lo && key < k_end;
        s[nt][i] = ok ? s[nt][i] * scale_log2 : -INFINITY;
        mx[i >> 1] = fmaxf(mx[i >> 1], s[nt][i]);
      }
  } else {
#pragma unroll
    for (int nt = 0; nt < 8; ++nt)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        s[nt][i] *= scale_log2;
        mx[i >> 1] = fmaxf(mx[i >> 1], s[nt][i]);
      }
  }
  float corr[2], msafe[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
    mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
    const float mn = fmaxf(m[r], mx[r]);
    msafe[r] = (mn == -INFINITY) ? 0.f : mn;
    corr[r] = exp2f(m[r] - msafe[r]);
    m[r] = mn;
    l[r] *= corr[r];
  }
  uint32_t pf[4][4];
#pragma unroll
  for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      s[nt][i] = exp2f(s[nt][i] - msafe[i >> 1]);
      l[i >> 1] += s[nt][i];
    }
    pf[nt >> 1][2 * (nt & 1)] = pack_bf16(s[nt][0], s[nt][1]);
    pf[nt >> 1][2 * (nt & 1) + 1] = pack_bf16(s[nt][2], s[nt][3]);
  }
#pragma unroll
  for (int nd = 0; nd < HD / 8; ++nd)
#pragma unroll
    for (int i = 0; i < 4; ++i) o[nd][i] *= corr[i >> 1];
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
    for (int nd = 0; nd < HD / 8; nd += 2) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, Vs + kv_off<HD, TMA_TILE>(16 * kk + 8 * (mat & 1) + r8, 8 * (nd + (mat >> 1))));
      mma_bf16(o[nd], pf[kk], b[0], b[1]);
      mma_bf16(o[nd + 1], pf[kk], b[2], b[3]);
    }
  }
}

// A CTA owns 128 rows (8 consumer warps x 16) of one (request, kv head) and walks the visible keys in 64-key
// tiles that a ninth warp fetches with TMA (page sizes 8 / 16 / 32 / 64) into a ring of stages.  Tiles wholly
// below every row's limit skip the mask; each warp stops at its own last visible tile.
constexpr int PREFILL_ROWS = 128;
constexpr int PREFILL_TMA_THREADS = 288;
constexpr int PREFILL_STAGES = 4;     // one CTA per SM (registers): a deep ring hides the load latency instead

template <int HD>
__global__ void __launch_bounds__(PREFILL_TMA_THREADS)
attn_prefill_tma_kernel(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* __restrict__ q,
                        long long q_row_stride, __nv_bfloat16* __restrict__ out, int* __restrict__ status,
                        const int* __restrict__ qo_indptr, const int* __restrict__ positions,
                        const int* __restrict__ kv_indptr, const int* __restrict__ kv_indices, int Hq, int Hkv,
                        int page_size, float scale_log2, int window, int min_q_long) {
  bspec::pdl_prologue(9);
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  constexpr int TILE_ELEMS = KT * HD;
  __nv_bfloat16* KV = reinterpret_cast<__nv_bfloat16*>(smem);                 // PREFILL_STAGES x (K tile, V tile)
  __nv_bfloat16* Qs = KV + PREFILL_STAGES * 2 * TILE_ELEMS;                   // [128][HD]
  uint64_t* full = reinterpret_cast<uint64_t*>(Qs + PREFILL_ROWS * HD);
  uint64_t* empty = full + PREFILL_STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty + PREFILL_STAGES);

  const int g = blockIdx.y, e = blockIdx.z;
  TileGeom t;
  if (!tile_geometry(t, qo_indptr, positions, e, g, Hq, Hkv)) return;
  if (t.q_len < min_q_long) return;
  const int n_row_tiles = (t.rows_total + PREFILL_ROWS - 1) / PREFILL_ROWS;
  if ((int)blockIdx.x >= n_row_tiles) return;
  const int row0 = (n_row_tiles - 1 - blockIdx.x) * PREFILL_ROWS;             // late (heavy) tiles first
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi_lo = row0 / t.G, qi_hi = min(t.q_len - 1, (row0 + PREFILL_ROWS - 1) / t.G);
  const int hi_key = t.pos0 + qi_hi;
  const int lo_key = window > 0 ? max(0, t.pos0 + qi_lo - window + 1) : 0;
  const int k_begin = (lo_key / KT) * KT, k_end = hi_key + 1;
  const int n_tiles = (k_end - k_begin + KT - 1) / KT;
  const int* table = kv_indices + kv_indptr[e];

  if (threadIdx.x == 0) {
    for (int s = 0; s < PREFILL_STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 8);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  if (warp == 8) {
    if (lane == 0) {
      const int first_pg = lo_key / page_size, last_pg = (k_end - 1) / page_size;
      const int pages_per_tile = KT / page_size;
      constexpr uint32_t tile_bytes = 2u * TILE_ELEMS * 2u;
      for (int it = 0; it < n_tiles; ++it) {
        const int s = it % PREFILL_STAGES;
        const uint32_t ph = (uint32_t)(it / PREFILL_STAGES) & 1u;
        if (!mbar_wait(empty + s, ph ^ 1u, abort_flag, status, 21)) break;
        __nv_bfloat16* Ks = KV + (size_t)s * 2 * TILE_ELEMS;
        mbar_expect_tx(full + s, tile_bytes);
        const int key0 = k_begin + it * KT;
        for (int pp = 0; pp < pages_per_tile; ++pp) {
          int pg = (key0 + pp * page_size) / page_size;
          pg = min(max(pg, first_pg), last_pg);
          const int page = table[pg];
          const int row_k = ((page * 2) * Hkv + g) * page_size;
          const int row_v = row_k + Hkv * page_size;
#pragma unroll
          for (int c = 0; c < HD / 64; ++c) {
            tma_load_2d(Ks + c * (KT * 64) + pp * page_size * 64, &kv_map, full + s, c * 64, row_k);
            tma_load_2d(Ks + TILE_ELEMS + c * (KT * 64) + pp * page_size * 64, &kv_map, full + s, c * 64, row_v);
          }
        }
      }
    }
    return;
  }

  // ---- consumers: warps 0..7
  const int wrow0 = row0 + 16 * warp;
  int lim[2], lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = wrow0 + (lane >> 2) + 8 * r;
    const int qi = row / t.G;
    lim[r] = row < t.rows_total ? t.pos0 + qi : -1;
    lo[r] = window > 0 ? max(0, t.pos0 + qi - window + 1) : 0;
  }
  const bool warp_live = wrow0 < t.rows_total;
  const int warp_hi = t.pos0 + min(t.q_len - 1, (wrow0 + 15) / t.G);          // last key any row of the warp sees
  const int warp_full = t.pos0 + wrow0 / t.G;                                 // keys <= this are seen by all its rows
  const int warp_lo = window > 0 ? t.pos0 + min(t.q_len - 1, (wrow0 + 15) / t.G) - window + 1 : 0;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

  // Q tile: 256 consumer threads load 128 rows
  {
    constexpr int CH = HD / 8;
    for (int idx = threadIdx.x; idx < PREFILL_ROWS * CH; idx += 256) {
      const int row = idx / CH, ch = idx - row * CH;
      const int r = row0 + row;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < t.rows_total) {
        const int qi = r / t.G, h = g * t.G + (r - qi * t.G);
        v = *reinterpret_cast<const uint4*>(q + (size_t)(t.q_begin + qi) * q_row_stride + (size_t)h * HD + ch * 8);
      }
      *reinterpret_cast<uint4*>(Qs + row * HD + ((ch ^ (row & 7)) << 3)) = v;
    }
  }
  asm volatile("bar.sync 1, 256;" ::: "memory");
  uint32_t qf[HD / 16][4];
  {
    const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
      ldmatrix_x4(qf[ks], Qs + swz<HD>(16 * warp + 8 * (mat & 1) + r8, 16 * ks + 8 * (mat >> 1)));
  }
  for (int it = 0; it < n_tiles; ++it) {
    const int s = it % PREFILL_STAGES;
    const uint32_t ph = (uint32_t)(it / PREFILL_STAGES) & 1u;
    if (!mbar_wait(full + s, ph, abort_flag, status, 22)) break;
    const __nv_bfloat16* Ks = KV + (size_t)s * 2 * TILE_ELEMS;
    const int key0 = k_begin + it * KT;
    if (warp_live && key0 <= warp_hi) {
      const bool need_mask = key0 + KT - 1 > warp_full || key0 < warp_lo || key0 + KT > k_end;
      block64<HD, true>(qf, Ks, Ks + TILE_ELEMS, key0, lim[0], lim[1], lo[0], lo[1], k_end, need_mask, scale_log2, m,
                        l, o);
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(empty + s);
  }
  if (*abort_flag || !warp_live) return;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = wrow0 + (lane >> 2) + 8 * r;
    if (row >= t.rows_total) continue;
    const int qi = row / t.G, h = g * t.G + (row - qi * t.G);
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    __nv_bfloat16* op = out + ((size_t)(t.q_begin + qi) * Hq + h) * HD;
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) {
      const int col = 8 * nd + 2 * (lane & 3);
      *reinterpret_cast<__nv_bfloat162*>(op + col) = __floats2bfloat162_rn(o[nd][2 * r] * inv, o[nd][2 * r + 1] * inv);
    }
  }
}

template <int HD> size_t prefill_tma_smem() {
  return 1024 + (size_t)PREFILL_STAGES * 2 * KT * HD * 2 + (size_t)PREFILL_ROWS * HD * 2 + 2 * PREFILL_STAGES * 8 + 64;
}

// ------------------------------------------------------------------------------------ prefill (64 rows per CTA)
template <int HD>
__global__ void __launch_bounds__(NTHREADS)
attn_prefill_kernel(const __nv_bfloat16* __restrict__ q, long long q_row_stride, __nv_bfloat16* __restrict__ out,
                    const __nv_bfloat16* __restrict__ cache, const int* __restrict__ qo_indptr,
                    const int* __restrict__ positions, const int* __restrict__ kv_indptr,
                    const int* __restrict__ kv_indices, int Hq, int Hkv, int page_size, float scale_log2, int window,
                    int min_q_long, long long n_pages) {
  bspec::pdl_prologue(9);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);           // [64][HD]
  __nv_bfloat16* KV = Qs + 64 * HD;                                        // 2 stages x (K, V)
  const int g = blockIdx.y, e = blockIdx.z;
  TileGeom t;
  if (!tile_geometry(t, qo_indptr, positions, e, g, Hq, Hkv)) return;
  if (t.q_len < min_q_long) return;
  // heavy (late) tiles first: they see the most keys
  const int n_row_tiles = (t.rows_total + 63) / 64;
  if ((int)blockIdx.x >= n_row_tiles) return;
  const int row0 = (n_row_tiles - 1 - blockIdx.x) * 64;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi_lo = row0 / t.G, qi_hi = min(t.q_len - 1, (row0 + 63) / t.G);
  const int hi_key = t.pos0 + qi_hi;
  const int lo_key = window > 0 ? max(0, t.pos0 + qi_lo - window + 1) : 0;
  const int k_begin = (lo_key / KT) * KT, k_end = hi_key + 1;
  const int* table = kv_indices + kv_indptr[e];
  const int wrow0 = row0 + 16 * warp;
  int lim[2], lo[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = wrow0 + (lane >> 2) + 8 * r;
    const int qi = row / t.G;
    lim[r] = row < t.rows_total ? t.pos0 + qi : -1;
    lo[r] = window > 0 ? max(0, t.pos0 + qi - window + 1) : 0;
  }
  // keys this warp's rows can see at all (skip tiles beyond its own last row)
  const int warp_hi = t.pos0 + min(t.q_len - 1, (wrow0 + 15) / t.G);
  const bool warp_live = wrow0 < t.rows_total;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o[i][j] = 0.f;

  load_q_tile<HD>(Qs, q, q_row_stride, t, row0, 64);
  const int n_tiles = (k_end - k_begin + KT - 1) / KT;
  load_kv_tile<HD>(KV, KV + KT * HD, cache, table, 0, k_begin, lo_key, k_end, page_size, Hkv, g, n_pages);
  cp_async_commit();
  __syncthreads();
  uint32_t qf[HD / 16][4];
  {
    const int mat = lane >> 3, r8 = lane & 7;
#pragma unroll
    for (int ks = 0; ks < HD / 16; ++ks)
      ldmatrix_x4(qf[ks], Qs + swz<HD>(16 * warp + 8 * (mat & 1) + r8, 16 * ks + 8 * (mat >> 1)));
  }
  for (int it = 0; it < n_tiles; ++it) {
    __nv_bfloat16* Ks = KV + (it & 1) * 2 * KT * HD;
    __nv_bfloat16* Vs = Ks + KT * HD;
    if (it + 1 < n_tiles) {
      __nv_bfloat16* Kn = KV + ((it + 1) & 1) * 2 * KT * HD;
      load_kv_tile<HD>(Kn, Kn + KT * HD, cache, table, 0, k_begin + (it + 1) * KT, lo_key, k_end, page_size, Hkv, g, n_pages);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = k_begin + it * KT;
    if (warp_live) {
#pragma unroll
      for (int kb = 0; kb < KT; kb += 16)
        if (key0 + kb <= warp_hi)
          block16<HD>(qf, Ks, Vs, kb, key0, lim[0], lim[1], lo[0], lo[1], k_end, scale_log2, m, l, o);
    }
    __syncthreads();
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
    l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = wrow0 + (lane >> 2) + 8 * r;
    if (row >= t.rows_total) continue;
    const int qi = row / t.G, h = g * t.G + (row - qi * t.G);
    const float inv = l[r] > 0.f ? 1.f / l[r] : 0.f;
    __nv_bfloat16* op = out + ((size_t)(t.q_begin + qi) * Hq + h) * HD;
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) {
      const int col = 8 * nd + 2 * (lane & 3);
      *reinterpret_cast<__nv_bfloat162*>(op + col) = __floats2bfloat162_rn(o[nd][2 * r] * inv, o[nd][2 * r + 1] * inv);
    }
  }
}

template <int HD> size_t decode_smem() {
  // Q tile, two K/V stages (reused by the combine: 4*16*HD + 128 floats, and by the join: 64*16 + 16 floats), table
  return (size_t)(16 + 4 * KT) * HD * 2 + (size_t)TBL_MAX * 4;
}
template <int HD> size_t prefill_smem() { return (size_t)(64 + 4 * KT) * HD * 2; }

template <int HD>
int launch(const __nv_bfloat16* q, long long q_row_stride, __nv_bfloat16* out, float* o_part, float* ml_part,
           int* tile_counters, int* status, long long kv_rows, const __nv_bfloat16* cache, const int* qo_indptr, const int* positions, const int* tok_entry,
           const int* kv_indptr, const int* kv_indices, int n_entries, int n_tokens, int max_q_len, int Hq, int Hkv,
           int page_size, float scale, int window, int n_splits, int max_q_short, int run_decode, int run_prefill,
           cudaStream_t stream, int balanced = 0, const int* kv_len = nullptr,
           long long check_pages = 0x7fffffffffffll) {
  const float scale_log2 = scale * 1.4426950408889634f;
  const int G = Hq / Hkv;
  // The opt-in to large shared memory and the resident-CTA count are facts of a device: set up once per device,
  // whichever thread gets there first.
  static std::once_flag once_dev[bspec::kMaxDevices];
  static int resident_dev[bspec::kMaxDevices] = {};
  const int cur_dev = bspec::current_device();
  std::call_once(once_dev[cur_dev], [cur_dev]() {
    cudaFuncSetAttribute(attn_decode_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_smem<HD>());
    cudaFuncSetAttribute(attn_decode_tma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)decode_tma_smem<HD>());
    cudaFuncSetAttribute(attn_decode_shares_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         (int)decode_shares_smem<HD>());
    cudaFuncSetAttribute(attn_decode_shares_kernel<HD>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    cudaFuncSetAttribute(attn_prefill_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)prefill_smem<HD>());
    if constexpr (HD <= 128)
      cudaFuncSetAttribute(attn_prefill_tma_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)prefill_tma_smem<HD>());
    int per_sm = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_decode_shares_kernel<HD>, DECODE_TMA_THREADS,
                                                  decode_shares_smem<HD>());
    resident_dev[cur_dev] = bspec::sm_count() * (per_sm > 0 ? per_sm : 1);
  });
  const int resident = resident_dev[cur_dev];
  if (run_decode) {
    const int short_q = max_q_len < max_q_short ? max_q_len : max_q_short;
    const int row_tiles = (short_q * G + 15) / 16;
    dim3 grid(n_splits, Hkv, n_entries * row_tiles);
    if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidConfiguration;
    bool launched = false;
    if (kv_rows > 0 && status != nullptr && page_size % 8 == 0 && KT % page_size == 0) {
      CUtensorMap kv_map;
      if (make_map_2d_bf16(&kv_map, cache, kv_rows, HD, page_size, 64)) {
       if (balanced && n_entries <= BAL_MAX_ENTRIES && n_splits >= 4 && n_splits <= 64 && n_tokens < (1 << 26)) {
        // equal shares of the tiles over as many CTAs as the device holds at once, then the join
        BSPEC_LAUNCH((attn_decode_shares_kernel<HD>), dim3(resident), DECODE_TMA_THREADS, decode_shares_smem<HD>(),
                     stream, kv_map, q, q_row_stride, out, o_part, ml_part, tile_counters, status, qo_indptr, positions,
                     kv_len, kv_indptr, kv_indices, n_entries, Hq, Hkv, page_size, scale_log2, window, n_splits,
                     short_q, row_tiles, max_q_short);
        launched = true;
       }
      }
      if (!launched && make_map_2d_bf16(&kv_map, cache, kv_rows, HD, page_size, 64)) {
        BSPEC_LAUNCH((attn_decode_tma_kernel<HD>), grid, DECODE_TMA_THREADS, decode_tma_smem<HD>(), stream, kv_map, q,
                     q_row_stride, out, o_part, ml_part, tile_counters, status, qo_indptr, positions, kv_indptr,
                     kv_indices, Hq, Hkv, page_size, scale_log2, window, n_splits, row_tiles, max_q_short);
        launched = true;
      }
    }
    if (!launched)
      BSPEC_LAUNCH((attn_decode_kernel<HD>), grid, NTHREADS, decode_smem<HD>(), stream,
                   q, q_row_stride, out, o_part, ml_part, tile_counters, cache, qo_indptr, positions, kv_indptr,
                   kv_indices, Hq, Hkv, page_size, scale_log2, window, n_splits, row_tiles, max_q_short, check_pages);
    const int err = (int)cudaGetLastError();
    if (err) return err;
  }
  if (run_prefill) {
    if (Hkv > 65535 || n_entries > 65535) return (int)cudaErrorInvalidConfiguration;
    bool launched = false;
    if constexpr (HD <= 128) {
     if (kv_rows > 0 && status != nullptr && page_size % 8 == 0 && KT % page_size == 0) {
      CUtensorMap kv_map;
      if (make_map_2d_bf16(&kv_map, cache, kv_rows, HD, page_size, 64)) {
        dim3 grid((max_q_len * G + PREFILL_ROWS - 1) / PREFILL_ROWS, Hkv, n_entries);
        BSPEC_LAUNCH((attn_prefill_tma_kernel<HD>), grid, PREFILL_TMA_THREADS, prefill_tma_smem<HD>(), stream, kv_map,
                     q, q_row_stride, out, status, qo_indptr, positions, kv_indptr, kv_indices, Hq, Hkv, page_size,
                     scale_log2, window, max_q_short + 1);
        launched = true;
      }
     }
    }
    if (!launched) {
      dim3 grid((max_q_len * G + 63) / 64, Hkv, n_entries);
      BSPEC_LAUNCH((attn_prefill_kernel<HD>), grid, NTHREADS, prefill_smem<HD>(), stream,
                   q, q_row_stride, out, cache, qo_indptr, positions, kv_indptr, kv_indices, Hq, Hkv, page_size,
                   scale_log2, window, max_q_short + 1, check_pages);
    }
    return (int)cudaGetLastError();
  }
  return 0;
}
}  // namespace

// Requests with q_len <= max_q_short go through the split-key kernel (if run_decode), the others through the
// 64-row kernel (if run_prefill).  n_splits (<= 64) > 1 needs scratch: o_part float32 [n_tokens * Hq * n_splits * hd],
// ml_part float32 [n_tokens * Hq * n_splits * 2] and tile_counters int32 [n_entries * Hkv * row tiles], which must
// be zero before the first launch and is left zero by every launch.  Returns cudaErrorInvalidValue for an
// unsupported head_dim.
// status: one int on the device (0 unless a bounded wait ran out); n_pages: pages of this cache layer (lets the
// split-key kernel load K/V through TMA; 0 keeps it on plain asynchronous copies).
// balanced != 0 (with n_pages > 0, 4 <= n_splits <= 64 and at most 512 requests): the short requests run on the
// kernel that gives every CTA an equal share of all key tiles.  n_splits is then the most partial results a row
// tile may get, and the scratch is indexed by request (o_part [n_entries * min(max_q_len, max_q_short) * Hq *
// n_splits * hd], ml_part likewise).  kv_len (may be null): [n_entries] each request's length after this step, which saves
// those kernels the dependent load of positions[qo_indptr[e]].  pages_in_all: pages of the cache layer whether or
// not n_pages is given (the checked build compares the page ids that the plain-copy kernels read with it; 0: unknown).
BSPEC_API int bspec_attention_bf16(const void* q, long long q_row_stride, void* out, float* o_part, float* ml_part,
                                   int* tile_counters, int* status, long long n_pages, const void* cache, const int* qo_indptr, const int* positions,
                                   const int* tok_entry, const int* kv_indptr, const int* kv_indices, int n_entries,
                                   int n_tokens, int max_q_len, int Hq, int Hkv, int hd, int page_size, float scale,
                                   int window, int n_splits, int max_q_short, int run_decode, int run_prefill,
                                   int balanced, const int* kv_len, long long pages_in_all, cudaStream_t stream) {
  if (n_entries <= 0 || n_tokens <= 0) return 0;
  if (Hq % Hkv != 0 || n_splits < 1 || n_splits > 64) return (int)cudaErrorInvalidValue;
#define GO(HDV)                                                                                                    \
  return launch<HDV>((const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, o_part, ml_part, tile_counters,   \
                     status, n_pages * 2 * Hkv * page_size, (const __nv_bfloat16*)cache, qo_indptr, positions, tok_entry, kv_indptr, kv_indices, n_entries, \
                     n_tokens, max_q_len, Hq, Hkv, page_size, scale, window, n_splits, max_q_short, run_decode,      \
                     run_prefill, stream, balanced, kv_len, pages_in_all > 0 ? pages_in_all : 0x7fffffffffffll)
  if (hd == 64) GO(64);
  if (hd == 128) GO(128);
  if (hd == 256) GO(256);
#undef GO
  return (int)cudaErrorInvalidValue;
}

// ---------------------------------------------------------------------------------------------------------------
// The same split-key decode attention for callers that cannot allocate: see attention_noalloc.h.
#include "attention_noalloc.h"
#include <stdio.h>

namespace {
// Scratch of the no-allocation entry point: [partial results | counters].  In host code this name is only a handle
// for cudaGetSymbolAddress; the kernels get the device address looked up below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[BSPEC_NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
void* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};
std::mutex g_noalloc_mutex;

int noalloc_refuse(int code, char* message, int message_len, const char* text) {
  if (message != nullptr && message_len > 0) snprintf(message, (size_t)message_len, "%s", text);
  return code;
}
}  // namespace

BSPEC_API int bspec_attention_decode_noalloc(const void* q, long long q_row_stride, void* out, const void* cache,
                                             const int* qo_indptr, const int* positions, const int* tok_entry,
                                             const int* kv_indptr, const int* kv_indices, int n_entries, int n_tokens,
                                             int max_q_len, int Hq, int Hkv, int head_dim, int page_size, float scale,
                                             int window, int n_splits, cudaStream_t stream, char* message,
                                             int message_len) {
  char text[256];
  if (n_entries <= 0 || n_tokens <= 0) return BSPEC_NOALLOC_OK;
  if (Hkv <= 0 || Hq % Hkv != 0 || (head_dim != 64 && head_dim != 128 && head_dim != 256) || n_splits < 1 ||
      n_splits > 64 || page_size < 1)
    return noalloc_refuse(BSPEC_NOALLOC_BAD_ARGUMENT, message, message_len,
                          "attention_decode_noalloc: head_dim must be 64/128/256, Hq a multiple of Hkv, 1 <= n_splits <= 64");
  const int G = Hq / Hkv;
  const int max_q_short = 16 / G > 1 ? 16 / G : 1;
  if (max_q_len > max_q_short) {
    snprintf(text, sizeof(text), "attention_decode_noalloc: serves requests of at most %d new tokens at this group size, got %d",
             max_q_short, max_q_len);
    return noalloc_refuse(BSPEC_NOALLOC_BAD_ARGUMENT, message, message_len, text);
  }
  const int row_tiles = (max_q_len * G + 15) / 16;
  const unsigned long long need_floats = (unsigned long long)n_tokens * Hq * n_splits * (head_dim + 2);
  const unsigned long long need_counters = (unsigned long long)n_entries * Hkv * row_tiles;
  if (n_splits > 1 && (need_floats > BSPEC_NOALLOC_MAX_PARTIAL_FLOATS || need_counters > BSPEC_NOALLOC_MAX_COUNTERS)) {
    snprintf(text, sizeof(text),
             "attention_decode_noalloc: needs %llu scratch floats and %llu counters, the built-in array holds %u and %u",
             need_floats, need_counters, BSPEC_NOALLOC_MAX_PARTIAL_FLOATS, BSPEC_NOALLOC_MAX_COUNTERS);
    return noalloc_refuse(BSPEC_NOALLOC_TOO_LARGE, message, message_len, text);
  }
  // Once per device, with that device current: the device address of the array.
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES)
    return noalloc_refuse(BSPEC_NOALLOC_SETUP_FAILED, message, message_len, "attention_decode_noalloc: no current device");
  void* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    if (g_noalloc_ptr[dev] == nullptr) {
      void* p = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
      if (e != cudaSuccess || p == nullptr) {
        snprintf(text, sizeof(text), "attention_decode_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                 cudaGetErrorString(e));
        return noalloc_refuse(BSPEC_NOALLOC_SETUP_FAILED, message, message_len, text);
      }
      g_noalloc_ptr[dev] = p;
    }
    base = g_noalloc_ptr[dev];
  }
  float* o_part = reinterpret_cast<float*>(base);
  float* ml_part = o_part + (size_t)n_tokens * Hq * n_splits * head_dim;
  int* counters = reinterpret_cast<int*>(reinterpret_cast<unsigned char*>(base) + (size_t)BSPEC_NOALLOC_MAX_PARTIAL_FLOATS * 4);
  if (n_splits > 1) {
    // the counters must start at zero whatever an earlier (possibly failed) call left behind
    const cudaError_t e = cudaMemsetAsync(counters, 0, (size_t)need_counters * sizeof(int), stream);
    if (e != cudaSuccess) return (int)e;
  }
#define GO(HDV)                                                                                                     \
  return launch<HDV>((const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, o_part, ml_part, counters, nullptr, \
                     0, (const __nv_bfloat16*)cache, qo_indptr, positions, tok_entry, kv_indptr, kv_indices,        \
                     n_entries, n_tokens, max_q_len, Hq, Hkv, page_size, scale, window, n_splits, max_q_short, 1, 0, \
                     stream)
  if (head_dim == 64) GO(64);
  if (head_dim == 128) GO(128);
  GO(256);
#undef GO
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_attention_bf16)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_attention_bf16)
