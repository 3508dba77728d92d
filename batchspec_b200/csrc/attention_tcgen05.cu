// Paged causal flash attention for long portions of prompts on the 5th-generation tensor cores (bfloat16,
// head_dim 128, page sizes 8 / 16 / 32 / 64).
//
// A CTA owns 128 rows, (token, query head of one kv group) pairs of one request and one kv head, and walks the
// visible keys in tiles of 128:
//   warp 0    TMA: K and V pages of the tile into a two-stage ring (one box per page and 64-column half,
//             128-byte swizzle, completion on an mbarrier);
//   warp 1    one thread issues tcgen05.mma:  S = Q K^T  (128 x 128 x 128, both operands K-major in shared memory)
//             into one of two S buffers in tensor memory, and  O += P V  (A = P in shared memory, B = V read
//             MN-major straight from the loaded pages) into the O accumulator in tensor memory;
//   warps 2-5 one thread per row: read its S row from tensor memory, scale, mask, online softmax in float32,
//             write P (bfloat16) into shared memory in the operand layout, rescale its O row in tensor memory
//             when the running maximum moved, and at the end normalise and store O.
// S of tile j+1 is computed while the softmax of tile j runs.  Every mbarrier wait is bounded; on expiry a code
// goes to `status`, all roles stop and the tensor memory is given back.
#include "common.cuh"
#include "tma.cuh"
#include <math.h>
using namespace bspec;

namespace {

constexpr int HD = 128;
constexpr int ROWS = 128;            // rows per CTA = accumulator lanes
constexpr int KT = 128;              // keys per tile
constexpr int STAGES = 2;
constexpr int THREADS = 192;
constexpr int SUB = ROWS * 64;       // elements of one [128][64] sub-tile (16 KB)
constexpr int TILE = 2 * SUB;        // a [128][128] operand tile (32 KB)

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(s32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
      ::"r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {          // 2^x on the special-function unit; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major operand tile: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(const void* tile) {
  const uint64_t addr = (uint64_t)((s32(tile) & 0x3FFFFu) >> 4);
  return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (V: rows = keys = K dimension, 64 contiguous head dims per 128-byte row): the next block of 64
// head dims is one sub-tile (16 KB) further, 8-key groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(const void* tile) {
  const uint64_t addr = (uint64_t)((s32(tile) & 0x3FFFFu) >> 4);
  return addr | ((uint64_t)((SUB * 2) >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// float32 accumulator, bfloat16 operands, M = 128, N = 128; b_mn: B operand is MN-major.
__device__ __forceinline__ uint32_t idesc(bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(128 >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}
// byte offset of 16-byte chunk `ch` (0..15) of row `row` in a [128][128] operand tile made of two swizzled sub-tiles
__device__ __forceinline__ int chunk_off(int row, int ch) {
  return (ch >> 3) * (SUB * 2) + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
}

struct Geom {
  int q_begin, q_len, pos0, G, rows_total;
};

__global__ void __launch_bounds__(THREADS)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap kv_map, const __nv_bfloat16* __restrict__ q,
                       long long q_row_stride, __nv_bfloat16* __restrict__ out, int* __restrict__ status,
                       const int* __restrict__ qo_indptr, const int* __restrict__ positions,
                       const int* __restrict__ kv_indptr, const int* __restrict__ kv_indices, int Hq, int Hkv,
                       int page_size, float scale_log2, int window, int min_q_long) {
  bspec::pdl_prologue(30);
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem);                  // [128][128]
  __nv_bfloat16* Ps = Qs + TILE;                                               // [128][128]
  __nv_bfloat16* KV = Ps + TILE;                                               // STAGES x (K tile, V tile)
  uint64_t* bars = reinterpret_cast<uint64_t*>(KV + STAGES * 2 * TILE);
  uint64_t* kv_full = bars;                 // [STAGES]
  uint64_t* kv_empty = bars + STAGES;       // [STAGES]
  uint64_t* s_full = bars + 2 * STAGES;     // [2]
  uint64_t* s_read = s_full + 2;            // [2]
  uint64_t* p_ready = s_read + 2;           // [1]
  uint64_t* pv_done = p_ready + 1;          // [1]
  uint64_t* q_ready = pv_done + 1;          // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int g = blockIdx.y, e = blockIdx.z;
  Geom t;
  t.q_begin = qo_indptr[e];
  t.q_len = qo_indptr[e + 1] - t.q_begin;
  if (t.q_len < min_q_long || t.q_len <= 0) return;
  t.pos0 = positions[t.q_begin];
  t.G = Hq / Hkv;
  t.rows_total = t.q_len * t.G;
  const int n_row_tiles = (t.rows_total + ROWS - 1) / ROWS;
  if ((int)blockIdx.x >= n_row_tiles) return;
  const int row0 = (n_row_tiles - 1 - blockIdx.x) * ROWS;                      // late (heavy) tiles first
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qi_lo = row0 / t.G, qi_hi = min(t.q_len - 1, (row0 + ROWS - 1) / t.G);
  const int hi_key = t.pos0 + qi_hi;
  const int lo_key = window > 0 ? max(0, t.pos0 + qi_lo - window + 1) : 0;
  const int k_begin = (lo_key / KT) * KT, k_end = hi_key + 1;
  const int n_tiles = (k_end - k_begin + KT - 1) / KT;
  const int* table = kv_indices + kv_indptr[e];

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(s_full + b, 1);
      mbar_init(s_read + b, 4);
    }
    mbar_init(p_ready, 4);
    mbar_init(pv_done, 1);
    mbar_init(q_ready, 4);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tmem_s[2] = {tmem, tmem + 128u};
  const uint32_t tmem_o = tmem + 256u;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      const int first_pg = lo_key / page_size, last_pg = (k_end - 1) / page_size;
      const int pages_per_tile = KT / page_size;
      for (int j = 0; j < n_tiles; ++j) {
        const int st = j % STAGES;
        const uint32_t ph = (uint32_t)(j / STAGES) & 1u;
        if (!mbar_wait(kv_empty + st, ph ^ 1u, abort_flag, status, 31)) break;
        __nv_bfloat16* Ks = KV + (size_t)st * 2 * TILE;
        mbar_expect_tx(kv_full + st, 2u * TILE * 2u);
        const int key0 = k_begin + j * KT;
        for (int pp = 0; pp < pages_per_tile; ++pp) {
          int pg = key0 / page_size + pp;
          pg = min(max(pg, first_pg), last_pg);
          const int page = table[pg];
          const int row_k = ((page * 2) * Hkv + g) * page_size;
          const int row_v = row_k + Hkv * page_size;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            tma_load_2d(Ks + c * SUB + pp * page_size * 64, &kv_map, kv_full + st, c * 64, row_k);
            tma_load_2d(Ks + TILE + c * SUB + pp * page_size * 64, &kv_map, kv_full + st, c * 64, row_v);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issue
    if (lane == 0) {
      const uint32_t id_s = idesc(false), id_o = idesc(true);
      bool ok = mbar_wait(q_ready, 0, abort_flag, status, 32);
      tc_fence_after();
      const uint64_t qdesc = desc_kmajor(Qs), pdesc = desc_kmajor(Ps);
      for (int j = 0; j <= n_tiles && ok; ++j) {
        if (j < n_tiles) {
          // S_j = Q K_j^T into S buffer j & 1
          const int st = j % STAGES, b = j & 1;
          ok = mbar_wait(kv_full + st, (uint32_t)(j / STAGES) & 1u, abort_flag, status, 33);
          if (ok && j >= 2) ok = mbar_wait(s_read + b, (uint32_t)((j >> 1) - 1) & 1u, abort_flag, status, 34);
          if (!ok) break;
          tc_fence_after();
          const uint64_t kdesc = desc_kmajor(KV + (size_t)st * 2 * TILE);
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint64_t off = (uint64_t)((ks >> 2) * ((SUB * 2) >> 4) + 2 * (ks & 3));
            tc_mma(tmem_s[b], qdesc + off, kdesc + off, id_s, ks > 0 ? 1u : 0u);
          }
          tc_commit(s_full + b);
          if (j < 6) bspec::trace_mark(130 + j, 0ull);                           // S_j issued
        }
        if (j >= 1) {
          // O += P_{j-1} V_{j-1}
          const int jj = j - 1, st = jj % STAGES;
          ok = mbar_wait(p_ready, (uint32_t)jj & 1u, abort_flag, status, 35);
          if (!ok) break;
          tc_fence_after();
          const uint64_t vdesc = desc_mnmajor(KV + (size_t)st * 2 * TILE + TILE);
#pragma unroll
          for (int kk = 0; kk < KT / 16; ++kk) {
            const uint64_t a_off = (uint64_t)((kk >> 2) * ((SUB * 2) >> 4) + 2 * (kk & 3));   // 16 keys = 32 bytes along P's rows
            const uint64_t b_off = (uint64_t)(kk * ((16 * 128) >> 4));                        // 16 keys = 16 rows of V
            tc_mma(tmem_o, pdesc + a_off, vdesc + b_off, id_o, (jj > 0 || kk > 0) ? 1u : 0u);
          }
          if (jj < 6) bspec::trace_mark(140 + jj, 0ull);                         // PV_jj issued
          tc_commit(kv_empty + st);       // K_{j-1} and V_{j-1} are no longer read
          tc_commit(pv_done);             // O holds tiles 0..j-1, P may be overwritten
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, one thread per row
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                        // row of the CTA tile = TMEM lane
    const int r = row0 + row;                                // row of the request
    const bool live = r < t.rows_total;
    const int qi = live ? r / t.G : 0;
    const int h = g * t.G + (live ? r - qi * t.G : 0);
    const int lim = live ? t.pos0 + qi : -1;
    const int lo = window > 0 ? max(0, t.pos0 + qi - window + 1) : 0;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    // Q tile: this thread copies its own row (16 chunks of 16 bytes) into the swizzled operand layout
    {
      const __nv_bfloat16* src = q + (size_t)(t.q_begin + qi) * q_row_stride + (size_t)h * HD;
      unsigned char* dst = reinterpret_cast<unsigned char*>(Qs);
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (live) v = *reinterpret_cast<const uint4*>(src + ch * 8);
        *reinterpret_cast<uint4*>(dst + chunk_off(row, ch)) = v;
      }
      fence_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_ready);
    }
    // m_ref: the maximum the probabilities and O are currently scaled by.  It follows the true running maximum
    // lazily: O and l are rescaled only when the maximum has grown by more than 8 (a factor 256, harmless in
    // float32 and bfloat16), which after the first tiles is rare.
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int b = j & 1;
      const unsigned long long t_a = (bspec::g_trace_buf != nullptr && j < 6) ? bspec::global_timer() : 0ull;
      ok = mbar_wait(s_full + b, (uint32_t)(j >> 1) & 1u, abort_flag, status, 36);
      if (!ok) break;
      tc_fence_after();
      if (threadIdx.x == 64 && j < 6) bspec::trace_mark(100 + j, t_a);          // waited for S_j
      const int key0 = k_begin + j * KT;
      const bool need_mask = key0 + KT - 1 > lim || key0 < lo || key0 + KT > k_end;
      // the whole S row into registers, then the S buffer is free for tile j + 2
      uint32_t sv[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tc_ld32(tmem_s[b] + lane_addr + 32u * c, sv[c]);
      tc_wait_ld();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_read + b);
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float sc = __uint_as_float(sv[c][i]) * scale_log2;
          if (need_mask) {
            const int key = key0 + 32 * c + i;
            if (!(key <= lim && key >= lo && key < k_end)) sc = -INFINITY;
          }
          sv[c][i] = __float_as_uint(sc);
          mx = fmaxf(mx, sc);
        }
      float corr = 1.f;
      if (mx > m_ref + 8.f || m_ref == -INFINITY) {           // (also the first tile that holds a visible key)
        const float m_new = fmaxf(m_ref, mx);
        corr = (m_new == -INFINITY) ? 1.f : ex2(m_ref - m_new);   // m_ref = -inf: O and l are still 0
        m_ref = m_new;
        l *= corr;
      }
      const float msafe = (m_ref == -INFINITY) ? 0.f : m_ref;
      // P may be overwritten, and O rescaled, only after the previous P V has completed
      const unsigned long long t_b = (bspec::g_trace_buf != nullptr && j < 6) ? bspec::global_timer() : 0ull;
      if (j >= 1) {
        ok = mbar_wait(pv_done, (uint32_t)(j - 1) & 1u, abort_flag, status, 37);
        if (!ok) break;
        tc_fence_after();
      }
      if (threadIdx.x == 64 && j < 6) bspec::trace_mark(110 + j, t_b);          // (max done) waited for PV_{j-1}
      unsigned char* pdst = reinterpret_cast<unsigned char*>(Ps);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = ex2(__uint_as_float(sv[c][i]) - msafe), p1 = ex2(__uint_as_float(sv[c][i + 1]) - msafe);
          l += p0 + p1;
          __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&hh);
        }
#pragma unroll
        for (int k4 = 0; k4 < 4; ++k4)
          *reinterpret_cast<uint4*>(pdst + chunk_off(row, 4 * c + k4)) =
              make_uint4(packed[4 * k4], packed[4 * k4 + 1], packed[4 * k4 + 2], packed[4 * k4 + 3]);
      }
      // rescale this row of O if its scale moved (the warp decides together: the TMEM access is warp-wide)
      if (j >= 1 && __any_sync(0xffffffffu, corr != 1.f)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tc_ld32(tmem_o + lane_addr + 32u * c, v);
          tc_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
          tc_st32(tmem_o + lane_addr + 32u * c, v);
        }
        tc_wait_st();
      }
      fence_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_ready);
      if (threadIdx.x == 64 && j < 6) bspec::trace_mark(120 + j, t_b);          // P written, arrived
    }
    // the last P V
    if (ok && n_tiles > 0) ok = mbar_wait(pv_done, (uint32_t)(n_tiles - 1) & 1u, abort_flag, status, 38);
    tc_fence_after();
    if (ok && n_tiles > 0) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* op = out + ((size_t)(t.q_begin + qi) * Hq + h) * HD;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tc_ld32(tmem_o + lane_addr + 32u * c, v);
        tc_wait_ld();
        if (live) {
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[8 * k4 + 2 * i]) * inv,
                                                        __uint_as_float(v[8 * k4 + 2 * i + 1]) * inv);
              w[i] = *reinterpret_cast<uint32_t*>(&hh);
            }
            *reinterpret_cast<uint4*>(op + 32 * c + 8 * k4) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
}

size_t smem_bytes() { return 1024 + (size_t)(2 + 2 * STAGES) * TILE * 2 + 16 * 8 + 64; }
}  // namespace

// Attention of the requests with at least `min_q_long` new tokens; the others are skipped (the split-key kernel
// serves them).  head_dim must be 128 and page_size one of 8 / 16 / 32 / 64; n_pages: pages of this cache layer.
// Returns cudaErrorInvalidValue for what it cannot do, so the caller can fall back.
BSPEC_API int bspec_attention_prefill_tc(const void* q, long long q_row_stride, void* out, int* status,
                                         long long n_pages, const void* cache, const int* qo_indptr,
                                         const int* positions, const int* kv_indptr, const int* kv_indices,
                                         int n_entries, int max_q_len, int Hq, int Hkv, int hd, int page_size,
                                         float scale, int window, int min_q_long, cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return 0;
  if (hd != HD || Hq % Hkv != 0 || page_size % 8 != 0 || KT % page_size != 0 || status == nullptr || n_pages <= 0)
    return (int)cudaErrorInvalidValue;
  if (Hkv > 65535 || n_entries > 65535) return (int)cudaErrorInvalidConfiguration;
  CUtensorMap kv_map;
  if (!make_map_2d_bf16(&kv_map, cache, n_pages * 2 * Hkv * page_size, HD, page_size, 64)) return (int)cudaErrorInvalidValue;
  static bool attr_set = false;
  if (!attr_set) {
    const cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem_bytes());
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int G = Hq / Hkv;
  dim3 grid((max_q_len * G + ROWS - 1) / ROWS, Hkv, n_entries);
  BSPEC_LAUNCH((attn_prefill_tc_kernel), grid, THREADS, smem_bytes(), stream, kv_map, (const __nv_bfloat16*)q,
               q_row_stride, (__nv_bfloat16*)out, status, qo_indptr, positions, kv_indptr, kv_indices, Hq, Hkv, page_size,
               scale * 1.4426950408889634f, window, min_q_long);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_attention_tcgen05)
