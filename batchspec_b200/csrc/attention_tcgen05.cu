// Paged causal flash attention for long portions of prompts on the 5th-generation tensor cores (bfloat16,
// head_dim 128, page sizes 8 / 16 / 32 / 64).
//
// One persistent CTA per SM works through items of 256 rows, (token, query head of one kv group) pairs of one
// request and one kv head, as two Q tiles of 128 rows with a softmax warpgroup each, and walks an item's visible
// keys in tiles of 64 (how the items are dealt and handed from role to role stands at the kernel):
//   warp 0    TMA: K and V pages of the key tile into a four-stage ring (one box per page and 64-column half,
//             128-byte swizzle, completion on an mbarrier), and the Q tiles;
//   warps 1, 10   one thread each issues tcgen05.mma for Q tile 0 / 1:  S = Q K^T  (128 x 64 x 128, operands
//             K-major in shared memory) into one of the tile's two S buffers in tensor memory, and  O += P V
//             (A = P read from tensor memory, B = V read MN-major straight from the loaded pages) into the
//             tile's O accumulator.  S runs two key tiles ahead; P V of tile j is issued the moment P_j is announced.
//   warps 2-5 / 6-9   Q tile 0 / 1, one thread per row: read its S row from tensor memory, scale, mask, online
//             softmax in float32 (two values per instruction where sm_100 has a packed form), write P (bfloat16)
//             back into tensor memory over the first half of the S buffer it came from, rescale its O row in tensor
//             memory when its scale moved, and at the end normalise and store O.
// The operands of a tcgen05.mma come out of shared memory at 128 bytes per clock, which is what such a product
// takes here (M = 128, K = 16: 48 clocks at N = 64, 64 at N = 128): with P in tensor memory the P V product
// fetches only V (32 clocks per instruction instead of 64), and the softmax threads write no shared memory.
// The softmax of a tile never waits for the tensor core in the steady state: S of the next key tile is ready.
// The issuing threads are two, in different warps, because they share their schedulers with softmax warps whose long runs of independent instructions keep
// them waiting some 300 cycles at every mbarrier they look at: with one thread for both Q tiles those waits and
// the (blocking) issues of both tiles stood in one line, and that line was the kernel's critical path.
// Tensor memory: 2 x 2 S buffers of 64 columns, 2 O accumulators of 128 (all 512 columns).  Every mbarrier wait is
// bounded; on expiry a code goes to `status`, all roles stop and the tensor memory is given back.
#include "common.cuh"
#include "tma.cuh"
#include <math.h>
using namespace bspec;

namespace {

constexpr int HD = 128;
constexpr int ROWS = 128;            // rows per Q tile = accumulator lanes
constexpr int QT = 2;                // Q tiles per CTA
constexpr int KT = 64;               // keys per tile
constexpr int STAGES = 4;
constexpr int MMA_WARP_1 = 2 + 4 * QT;                 // the second Q tile's MMA warp: after the softmax warps
constexpr int THREADS = 32 * (3 + 4 * QT);
constexpr int SUBQ = ROWS * 64;      // elements of a [128][64] sub-tile (16 KB): Q halves, P
constexpr int SUBK = KT * 64;        // elements of a [64][64] sub-tile (8 KB): K and V halves
constexpr int QTILE = 2 * SUBQ;      // [128][128] Q tile
constexpr int KTILE = 2 * SUBK;      // [64][128] K (or V) tile

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
// the A operand read from tensor memory (rows on the lanes, two bfloat16 per 32-bit column)
__device__ __forceinline__ void tc_mma_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accum) : "memory");
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
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
      ::"r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ float ex2(float x) {          // 2^x on the special-function unit; 2^-inf = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two float32 operations per instruction (sm_100 has packed forms of add, mul and fma) and a maximum of three:
// the softmax is bound by the number of instructions it issues, not by the arithmetic pipes.
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major operand tile: rows of 128 bytes, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_kmajor(const void* tile) {
  const uint64_t addr = (uint64_t)((s32(tile) & 0x3FFFFu) >> 4);
  return addr | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand (V: rows = keys = K dimension, 64 contiguous head dims per 128-byte row): the next block of 64
// head dims is one sub-tile (8 KB) further, 8-key groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t desc_mnmajor(const void* tile) {
  const uint64_t addr = (uint64_t)((s32(tile) & 0x3FFFFu) >> 4);
  return addr | ((uint64_t)((SUBK * 2) >> 4) << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// float32 accumulator, bfloat16 operands, M = 128, N = n; b_mn: B operand is MN-major.
__device__ __forceinline__ uint32_t idesc(int n, bool b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (b_mn ? (1u << 16) : 0u) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

struct Geom {
  int q_begin, q_len, pos0, G, rows_total;
};

// One work item: 256 rows (two Q tiles) of one request and one kv head.
struct Item {
  Geom t;
  int e, g, row0;
  int lo_key, k_begin, k_end, n_tiles;
  int n_kt[QT], k_end_t[QT];
  const int* table;
};

// The launch's items in the order they are dealt: kv head fastest, then request, then the request's 256-row blocks
// from its last (most keys) to its first.  Returns false for an index that names no work (a request of the other
// kernel, or fewer rows than the longest request).
__device__ __forceinline__ bool load_item(Item& it, int idx, int Hq, int Hkv, int n_entries, int window,
                                          int page_size, int min_q_long, const int* __restrict__ qo_indptr,
                                          const int* __restrict__ positions, const int* __restrict__ kv_indptr,
                                          const int* __restrict__ kv_indices) {
  const int g = idx % Hkv, ez = idx / Hkv;
  const int e = ez % n_entries, z = ez / n_entries;
  Geom& t = it.t;
  t.q_begin = qo_indptr[e];
  t.q_len = qo_indptr[e + 1] - t.q_begin;
  if (t.q_len < min_q_long || t.q_len <= 0) return false;
  t.G = Hq / Hkv;
  t.rows_total = t.q_len * t.G;
  const int n_cta_tiles = (t.rows_total + QT * ROWS - 1) / (QT * ROWS);
  if (z >= n_cta_tiles) return false;
  t.pos0 = positions[t.q_begin];
  it.e = e;
  it.g = g;
  it.row0 = (n_cta_tiles - 1 - z) * QT * ROWS;
  const int qi_lo = it.row0 / t.G;
  it.lo_key = window > 0 ? max(0, t.pos0 + qi_lo - window + 1) : 0;
  it.k_begin = (it.lo_key / KT) * KT;
#pragma unroll
  for (int tt = 0; tt < QT; ++tt) {
    const int r_first = it.row0 + tt * ROWS;
    if (r_first < t.rows_total) {
      const int qi_hi = min(t.q_len - 1, (r_first + ROWS - 1) / t.G);
      it.k_end_t[tt] = t.pos0 + qi_hi + 1;
      it.n_kt[tt] = (it.k_end_t[tt] - it.k_begin + KT - 1) / KT;
    } else {
      it.k_end_t[tt] = it.k_begin;
      it.n_kt[tt] = 0;
    }
  }
  it.n_tiles = max(it.n_kt[0], it.n_kt[1]);
  it.k_end = max(it.k_end_t[0], it.k_end_t[1]);
  it.table = kv_indices + kv_indptr[e];
  return true;
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(s32(dst)), "l"(map), "r"(s32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}

constexpr int ITEM_RING = 8;

// A persistent CTA per SM.  Items are handed out heaviest first from a counter in global memory (CTA c starts with
// item c): the producer warp draws the CTA's next item while the current one runs, looks up its lengths and
// positions (three dependent loads) and leaves the finished description in a small ring in shared memory, from
// which the other roles take it; an item with n_tiles < 0 ends the list.  The producer is at most three key tiles
// (so at most three items) ahead of the MMA threads and those at most two ahead of the softmax threads, and every
// item has at least one key tile: eight slots are never overrun.
// The roles keep their own running counts of key tiles and items, from which every mbarrier's stage and phase
// follow; nothing but the tensor memory allocation is shared between items, so the next item's keys and queries
// are fetched, and its first two S tiles computed, while the softmax threads still finish and store the item
// before.  The CTA that leaves last puts the counter back to zero for the next launch.
__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap kv_map, const __grid_constant__ CUtensorMap q_map,
                       const __nv_bfloat16* __restrict__ q, long long q_row_stride, __nv_bfloat16* __restrict__ out,
                       int* __restrict__ status, const int* __restrict__ qo_indptr, const int* __restrict__ positions,
                       const int* __restrict__ kv_indptr, const int* __restrict__ kv_indices, int Hq, int Hkv,
                       int n_entries, int n_items, int page_size, float scale_log2, int window, int min_q_long,
                       int q_by_tma, int* __restrict__ work) {
  // The step's lengths, positions and block tables were uploaded before its first kernel: the set-up below and the
  // look-up of the CTA's first item read nothing that the kernel before this one writes, so they run under its
  // tail; q, the new tokens' keys and `out` are touched only after the wait.
  const unsigned long long t_trace = bspec::g_trace_buf != nullptr ? bspec::global_timer() : 0ull;
  bspec::pdl_launch_dependents();
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem);                  // QT x [128][128]
  __nv_bfloat16* Os = Qs + QT * QTILE;                                         // QT x [128][64]: O on its way out
  __nv_bfloat16* KV = Os + QT * SUBQ;                                          // STAGES x (K tile, V tile)
  uint64_t* bars = reinterpret_cast<uint64_t*>(KV + STAGES * 2 * KTILE);
  uint64_t* kv_full = bars;                        // [STAGES]
  uint64_t* kv_empty = kv_full + STAGES;           // [STAGES]
  uint64_t* s_full = kv_empty + STAGES;            // [QT][2]
  uint64_t* p_ready = s_full + 2 * QT;             // [QT][2]
  uint64_t* pv_done = p_ready + 2 * QT;            // [QT][2]
  uint64_t* q_ready = pv_done + 2 * QT;            // [QT]  the item's Q tile is in shared memory
  uint64_t* q_free = q_ready + QT;                 // [QT]  every S product of the item has read it
  uint64_t* o_free = q_free + QT;                  // [QT]  the item's O has been read out of tensor memory
  uint64_t* item_full = o_free + QT;               // [ITEM_RING]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(item_full + ITEM_RING);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  Item* items = reinterpret_cast<Item*>(tmem_slot + 4);     // [ITEM_RING]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, QT);      // one arrival per Q tile's MMA thread
    }
    for (int i = 0; i < 2 * QT; ++i) {
      mbar_init(s_full + i, 1);
      mbar_init(p_ready + i, 4);
      mbar_init(pv_done + i, 1);
    }
    for (int i = 0; i < QT; ++i) {
      mbar_init(q_ready + i, q_by_tma ? 1 : 4);
      mbar_init(q_free + i, 1);
      mbar_init(o_free + i, 4);
    }
    for (int i = 0; i < ITEM_RING; ++i) mbar_init(item_full + i, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  Item it;
  bool first_found = false;
  if (warp == 0)
    first_found = load_item(it, blockIdx.x, Hq, Hkv, n_entries, window, page_size, min_q_long, qo_indptr, positions,
                            kv_indptr, kv_indices);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  bspec::pdl_wait();
  bspec::trace_record(30, t_trace);
  uint32_t item_no = 0;          // items this role has taken from the ring
  // the other roles' way to the next item: false at the end of the list (or when a wait gave up)
#define NEXT_ITEM() (mbar_wait(item_full + item_no % ITEM_RING, (item_no / ITEM_RING) & 1u, abort_flag, status, 41) && \
                     (it = items[item_no % ITEM_RING], ++item_no, it.n_tiles >= 0))

  if (warp == 0) {
    // ------------------------------------------------------------------ producer
    // Lane p fetches page p of every key tile (at most 8 pages per tile): it reads the page's table entry one
    // tile ahead, so no copy waits on a table lookup, and issues that page's four copies itself.  Lane 0 also
    // fetches the item's Q tiles (two boxes of [tokens][heads of the group][64] each) once the S products of the
    // item before have all read theirs.
    const int pages_per_tile = KT / page_size;
    const bool mine = lane < pages_per_tile;
    uint32_t kv_no = 0, q_no[QT] = {0, 0};
    int ok = 1;
    int cand = blockIdx.x;       // the next index to look at: the CTA's own first, then what the counter gives
    bool first = true;
    while (ok) {
      // The next index that names work.  It is drawn only now, when the item before has been fetched to its last
      // key tile (the other roles are about three tiles from its end): drawn earlier, the items would go to the
      // CTAs in the order they started, not in the order they come free, and the heaviest would get a second one.
      bool found = false;
      auto draw = [&]() {
        int drawn = 0;
        if (lane == 0) drawn = atomicAdd(work, 1) + (int)gridDim.x;
        cand = __shfl_sync(0xffffffffu, drawn, 0);
      };
      if (first) {                                   // the CTA's own index was looked up before the set-up barrier
        first = false;
        found = first_found;
        if (!found) draw();
      }
      while (cand < n_items && !found) {
        found = load_item(it, cand, Hq, Hkv, n_entries, window, page_size, min_q_long, qo_indptr, positions, kv_indptr,
                          kv_indices);
        if (!found) draw();
      }
      if (!found) it.n_tiles = -1;
      if (lane == 0) {
        items[item_no % ITEM_RING] = it;
        mbar_arrive(item_full + item_no % ITEM_RING);
      }
      ++item_no;
      if (!found) break;
      if (q_by_tma) {
        if (lane == 0) {
#pragma unroll
          for (int tt = 0; tt < QT; ++tt) {
            if (it.n_kt[tt] == 0) continue;
            if (q_no[tt] > 0 && !mbar_wait(q_free + tt, (q_no[tt] - 1) & 1u, abort_flag, status, 39)) { ok = 0; break; }
            mbar_expect_tx(q_ready + tt, (uint32_t)QTILE * 2u);
            const int tok0 = it.t.q_begin + (it.row0 + tt * ROWS) / it.t.G;
            tma_load_3d(Qs + tt * QTILE, &q_map, q_ready + tt, 0, it.g * it.t.G, tok0);
            tma_load_3d(Qs + tt * QTILE + SUBQ, &q_map, q_ready + tt, 64, it.g * it.t.G, tok0);
          }
        }
#pragma unroll
        for (int tt = 0; tt < QT; ++tt) q_no[tt] += it.n_kt[tt] > 0 ? 1u : 0u;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
      const int first_pg = it.lo_key / page_size, last_pg = max(first_pg, (it.k_end - 1) / page_size);
      auto page_of = [&](int j) -> int {
        int pg = (it.k_begin + j * KT) / page_size + lane;
        pg = min(max(pg, first_pg), last_pg);
        return it.table[pg];
      };
      int page_next = mine ? page_of(0) : 0;
      for (int j = 0; j < it.n_tiles; ++j, ++kv_no) {
        const int st = kv_no % STAGES;
        const uint32_t ph = (kv_no / STAGES) & 1u;
        const int page = page_next;
        if (mine && j + 1 < it.n_tiles) page_next = page_of(j + 1);
        if (lane == 0) {
          ok = mbar_wait(kv_empty + st, ph ^ 1u, abort_flag, status, 31) ? 1 : 0;
          if (ok) mbar_expect_tx(kv_full + st, 2u * KTILE * 2u);
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        if (mine) {
          __nv_bfloat16* Ks = KV + (size_t)st * 2 * KTILE;
          const int row_k = ((page * 2) * Hkv + it.g) * page_size;
          const int row_v = row_k + Hkv * page_size;
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            tma_load_2d(Ks + c * SUBK + lane * page_size * 64, &kv_map, kv_full + st, c * 64, row_k);
            tma_load_2d(Ks + KTILE + c * SUBK + lane * page_size * 64, &kv_map, kv_full + st, c * 64, row_v);
          }
        }
      }
      int drawn = 0;
      if (lane == 0) drawn = atomicAdd(work, 1) + (int)gridDim.x;
      cand = __shfl_sync(0xffffffffu, drawn, 0);
    }
  } else if (warp == 1 || warp == MMA_WARP_1) {
    // ------------------------------------------------------------------ MMA issue, one thread per Q tile
    // A wait on an mbarrier costs this thread some 300 cycles even when the barrier is long complete, and its
    // tcgen05.mma instructions block while the tensor core's queue is full: with one thread for both Q tiles the
    // waits and the issues of the two tiles stood in one line and that line was the kernel's critical path.  Each
    // Q tile now has its own issuing thread (in different warps); the tensor core takes from both.
    const int tt = warp == 1 ? 0 : 1;
    if (lane == 0) {
      const uint32_t id_s = idesc(KT, false), id_o = idesc(HD, true);
      const uint64_t qdesc = desc_kmajor(Qs + tt * QTILE);
      uint32_t kv_base = 0;      // key tiles of the items before this one (all of them pass through the ring)
      uint32_t sq = 0;           // key tiles of this Q tile before this item: the S buffers (and P in them) alternate with it
      uint32_t n_mine = 0;       // items before this one in which this Q tile had rows
      bool ok = true;
      while (ok && NEXT_ITEM()) {
        const int my_tiles = it.n_kt[tt], n_tiles = it.n_tiles;
        if (my_tiles > 0) ok = mbar_wait(q_ready + tt, n_mine & 1u, abort_flag, status, 32);
        tc_fence_after();
        // S_j = Q K_j^T into the S buffer of the tile's running number
        auto issue_s = [&](int j) -> bool {
          const uint32_t kn = kv_base + (uint32_t)j, bf = (sq + (uint32_t)j) & 1u;
          const int st = kn % STAGES;
          if (!mbar_wait(kv_full + st, (kn / STAGES) & 1u, abort_flag, status, 33)) return false;
          // The buffer was last used by the key tile two before this one.  Its softmax read S out of it before it
          // announced P of that tile, and this thread has seen that announcement (it issued that tile's P V,
          // also across the end of an item): no wait here.
          tc_fence_after();
          const uint64_t kdesc = desc_kmajor(KV + (size_t)st * 2 * KTILE);
          const uint32_t d = tmem + (uint32_t)(tt * 128) + bf * 64u;
#pragma unroll
          for (int ks = 0; ks < HD / 16; ++ks) {
            const uint64_t a_off = (uint64_t)((ks >> 2) * ((SUBQ * 2) >> 4) + 2 * (ks & 3));
            const uint64_t b_off = (uint64_t)((ks >> 2) * ((SUBK * 2) >> 4) + 2 * (ks & 3));
            tc_mma(d, qdesc + a_off, kdesc + b_off, id_s, ks > 0 ? 1u : 0u);
          }
          tc_commit(s_full + 2 * tt + bf);
          if (j == my_tiles - 1) tc_commit(q_free + tt);     // the item's last S: its Q tile may be replaced
          return true;
        };
        // S runs two key tiles ahead of P V (two S buffers per Q tile, four K/V stages)
        for (int j = 0; j < 2 && j < my_tiles && ok; ++j) ok = issue_s(j);
        for (int j = 0; j < n_tiles && ok; ++j) {
          const uint32_t kn = kv_base + (uint32_t)j;
          const int st = kn % STAGES;
          if (j >= my_tiles) {
            // Key tiles that only the other Q tile sees: this tile's share of the release of their stage, given once
            // the tile has arrived (so that two of these cannot fall into one phase of the stage's barrier).
            ok = mbar_wait(kv_full + st, (kn / STAGES) & 1u, abort_flag, status, 33);
            if (ok) mbar_arrive(kv_empty + st);
            continue;
          }
          // O += P_j V_j, as soon as the softmax has written P_j: the softmax of tile j + 1 then never waits for it
          // (its P goes to the other buffer), and the tensor core has S of tiles j + 1 and j + 2 to work on meanwhile
          const uint32_t pn = sq + (uint32_t)j, bf = pn & 1u;
          ok = mbar_wait(p_ready + 2 * tt + bf, (pn >> 1) & 1u, abort_flag, status, 35);
          if (!ok) break;
          // the first P V of an item overwrites O: the softmax threads must have read the item before out of it
          if (j == 0 && n_mine > 0) {
            ok = mbar_wait(o_free + tt, (n_mine - 1) & 1u, abort_flag, status, 40);
            if (!ok) break;
          }
          tc_fence_after();
          const uint32_t p_tmem = tmem + (uint32_t)(tt * 128) + bf * 64u;     // P: the first 32 columns of its S buffer
          const uint64_t vdesc = desc_mnmajor(KV + (size_t)st * 2 * KTILE + KTILE);
          const uint32_t d = tmem + (uint32_t)(256 + tt * 128);
#pragma unroll
          for (int kk = 0; kk < KT / 16; ++kk)          // 16 keys: 8 columns of P, 16 rows of V
            tc_mma_a_tmem(d, p_tmem + (uint32_t)(8 * kk), vdesc + (uint64_t)(kk * ((16 * 128) >> 4)), id_o,
                          (j > 0 || kk > 0) ? 1u : 0u);
          tc_commit(pv_done + 2 * tt + bf);              // O holds key tiles 0..j
          tc_commit(kv_empty + st);                      // this Q tile no longer reads K_j and V_j
          // S of key tile j + 2 (its K was fetched into the stage that the P V of tile j - 1 released)
          if (j + 2 < my_tiles) ok = issue_s(j + 2);
        }
        kv_base += (uint32_t)n_tiles;
        sq += (uint32_t)my_tiles;
        n_mine += my_tiles > 0 ? 1u : 0u;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, one thread per row
    const int tt = (warp - 2) >> 2;                          // Q tile of this warpgroup
    const int quad = warp & 3;                               // TMEM lanes this warp may touch
    const int row = quad * 32 + lane;                        // row of the Q tile = TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t tmem_o = tmem + (uint32_t)(256 + tt * 128) + lane_addr;
    unsigned char* stage = reinterpret_cast<unsigned char*>(Os + tt * SUBQ) + row * 128;   // this thread's row
    uint32_t sq = 0;             // key tiles of this Q tile before this item
    bool ok = true;
    while (ok && NEXT_ITEM()) {
      const int my_tiles = it.n_kt[tt];
      if (my_tiles == 0) continue;
      const Geom& t = it.t;
      const int g = it.g;
      const int r = it.row0 + tt * ROWS + row;               // row of the request
      const bool live = r < t.rows_total;
      const int qi = live ? r / t.G : 0;
      const int h = g * t.G + (live ? r - qi * t.G : 0);
      const int lim = live ? t.pos0 + qi : -1;
      const int lo = window > 0 ? max(0, t.pos0 + qi - window + 1) : 0;
      const int my_k_end = it.k_end_t[tt];
      if (!q_by_tma) {
        // Q tile: this thread copies its own row (16 chunks of 16 bytes) into the swizzled operand layout.  The
        // S products of the item before are long complete: this thread has waited for that item's last P V,
        // which the same thread issued after them.
        const __nv_bfloat16* src = q + (size_t)(t.q_begin + qi) * q_row_stride + (size_t)h * HD;
        unsigned char* dst = reinterpret_cast<unsigned char*>(Qs + tt * QTILE);
#pragma unroll
        for (int ch = 0; ch < 16; ++ch) {
          uint4 v = make_uint4(0, 0, 0, 0);
          if (live) v = *reinterpret_cast<const uint4*>(src + ch * 8);
          *reinterpret_cast<uint4*>(dst + (ch >> 3) * (SUBQ * 2) + row * 128 + (((ch & 7) ^ (row & 7)) << 4)) = v;
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_ready + tt);
      }
      // m_ref: the maximum the probabilities and O are currently scaled by.  It follows the true running maximum
      // lazily: it is looked for again only when a tile's probabilities sum to more than 2^14, and O and l are then
      // rescaled if it has grown by more than 8; after the first tiles of an item that is rare.
      float m_ref = -INFINITY, l = 0.f;
      for (int j = 0; j < my_tiles && ok; ++j) {
        const uint32_t n = sq + (uint32_t)j, b = n & 1u;
        ok = mbar_wait(s_full + 2 * tt + b, (n >> 1) & 1u, abort_flag, status, 36);
        if (!ok) break;
        tc_fence_after();
        const int key0 = it.k_begin + j * KT;
        const bool need_mask = key0 + KT - 1 > lim || key0 < lo || key0 + KT > my_k_end;
        // the whole S row into registers, then the S buffer is free for the key tile after next
        uint32_t sv[2][32];
        const uint32_t s_addr = tmem + (uint32_t)(tt * 128) + b * 64u + lane_addr;
        tc_ld32(s_addr, sv[0]);
        tc_ld32(s_addr + 32u, sv[1]);
        tc_wait_ld();
        // P = 2^(scale * S - m) for the row, its sum returned; scaling and the row sum handle two values per
        // instruction (fma/add.f32x2), the exponentials all go to the special-function unit (masked scores are -inf
        // and come out as exactly 0).  Each half of P goes back into tensor memory as soon as it is complete, over
        // the first half of the S buffer this thread has just read, so that the store's latency runs under the
        // second half's arithmetic: the P V product takes its A operand from there.  What the columns held before
        // (P of the key tile two before this one) was read by a product that was issued, and so completed, before
        // this S.  The stores are warp-wide: every path to this point is taken by the whole warp.
        auto exponentials = [&](float neg_m) -> float {
          uint32_t packed[32];
          const uint64_t scale2 = pack2(scale_log2, scale_log2), neg_m2 = pack2(neg_m, neg_m);
          uint64_t l2[2] = {pack2(0.f, 0.f), pack2(0.f, 0.f)};
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float p0, p1;
              unpack2(fma2(pack2(__uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1])), scale2, neg_m2), p0, p1);
              p0 = ex2(p0);
              p1 = ex2(p1);
              l2[(i >> 1) & 1] = add2(l2[(i >> 1) & 1], pack2(p0, p1));
              __nv_bfloat162 hh = __floats2bfloat162_rn(p0, p1);
              packed[16 * c + (i >> 1)] = *reinterpret_cast<uint32_t*>(&hh);
            }
            tc_st16(s_addr + 16u * c, packed + 16 * c);
          }
          float la, lb;
          unpack2(add2(l2[0], l2[1]), la, lb);
          return la + lb;
        };
        // Most tiles need no new maximum: the probabilities are formed with the maximum the row is scaled by already,
        // and their sum tells whether that was safe.  A sum of at most 2^14 bounds every one of them by 2^14, which
        // float32 and bfloat16 carry without loss; a larger one (or infinity) sends the warp through the full
        // path below, as do the first tile of an item and tiles that need a mask.
        float corr = 1.f, row_sum = 0.f;
        bool full_path = __any_sync(0xffffffffu, need_mask || m_ref == -INFINITY);
        if (!full_path) {
          row_sum = exponentials(-m_ref);
          full_path = __any_sync(0xffffffffu, !(row_sum <= 16384.f));
          if (full_path) tc_wait_st();          // the stores above land before the ones that replace them
        }
        if (full_path) {
          // maximum of the raw scores (the scale is positive), masked entries set to -inf in place
          float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
          if (need_mask) {                   // a tile on the diagonal, at the window's edge or at the end of the keys
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i = 0; i < 32; ++i) {
                const int key = key0 + 32 * c + i;
                if (!(key <= lim && key >= lo && key < my_k_end)) sv[c][i] = 0xff800000u;      // -inf
                mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(sv[c][i]));
              }
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c)
#pragma unroll
              for (int i = 0; i < 32; i += 2)
                mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
          }
          const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
          if (mx > m_ref + 8.f || m_ref == -INFINITY) {         // (also the first tile that holds a visible key)
            const float m_new = fmaxf(m_ref, mx);
            corr = (m_new == -INFINITY) ? 1.f : ex2(m_ref - m_new);   // m_ref = -inf: O and l are still 0
            m_ref = m_new;
            l *= corr;
          }
          __syncwarp();
          row_sum = exponentials((m_ref == -INFINITY) ? 0.f : -m_ref);
        }
        l += row_sum;
        // rescale this row of O if its scale moved (the warp decides together: the TMEM access is warp-wide); the
        // P V of key tile j - 1 must have completed before O is touched
        if (j >= 1 && __any_sync(0xffffffffu, corr != 1.f)) {
          ok = mbar_wait(pv_done + 2 * tt + (b ^ 1u), ((n - 1) >> 1) & 1u, abort_flag, status, 37);
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tc_ld32(tmem_o + 32u * c, v);
            tc_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
            tc_st32(tmem_o + 32u * c, v);
          }
        }
        tc_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_ready + 2 * tt + b);
      }
      // the last P V
      const uint32_t n_last = sq + (uint32_t)my_tiles - 1u;
      if (ok) ok = mbar_wait(pv_done + 2 * tt + (n_last & 1u), (n_last >> 1) & 1u, abort_flag, status, 38);
      tc_fence_after();
      if (ok) {
        // O: tensor memory -> registers (normalised, bfloat16) -> this warp's own 32 rows of a staging tile in
        // shared memory -> global memory in runs of 128 bytes, 8 lanes per row, 64 columns at a time.  A thread
        // storing its own row would touch 32 different lines per instruction.
        const float inv = l > 0.f ? 1.f / l : 0.f;
        const unsigned char* wbase = reinterpret_cast<const unsigned char*>(Os + tt * SUBQ) + (quad * 32) * 128;
        const int sub = lane >> 3, ch8 = lane & 7;                   // four rows per pass, 8 chunks of a half row
        const int r_warp = it.row0 + tt * ROWS + quad * 32;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            const int c = 2 * half + c2;
            uint32_t v[32];
            tc_ld32(tmem_o + 32u * c, v);
            tc_wait_ld();
            if (c == 3) {
              // O is in registers: the next item's first P V may overwrite it
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(o_free + tt);
            }
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              uint32_t w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 hh = __floats2bfloat162_rn(__uint_as_float(v[8 * k4 + 2 * i]) * inv,
                                                          __uint_as_float(v[8 * k4 + 2 * i + 1]) * inv);
                w[i] = *reinterpret_cast<uint32_t*>(&hh);
              }
              const int ch = 4 * c2 + k4;                            // 16-byte chunk of the 64-column half
              *reinterpret_cast<uint4*>(stage + ((ch ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
            }
          }
          __syncwarp();
#pragma unroll 4
          for (int i = 0; i < 8; ++i) {
            const int rl = 4 * i + sub, rr = r_warp + rl;
            if (rr < t.rows_total) {
              const uint4 v4 = *reinterpret_cast<const uint4*>(wbase + rl * 128 + ((ch8 ^ (rl & 7)) << 4));
              const int qr = rr / t.G, hr = g * t.G + (rr - qr * t.G);
              *reinterpret_cast<uint4*>(out + ((size_t)(t.q_begin + qr) * Hq + hr) * HD + 64 * half + 8 * ch8) = v4;
            }
          }
          __syncwarp();                                              // before the rows are written again
        }
      }
      sq += (uint32_t)my_tiles;
    }
  }
#undef NEXT_ITEM
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
  }
  // every CTA has drawn its last index by now: the last one to leave resets the two counters
  if (threadIdx.x == 0 && atomicAdd(work + 1, 1) == (int)gridDim.x - 1) {
    work[0] = 0;
    work[1] = 0;
  }
}

size_t smem_bytes() {
  return 1024 + (size_t)(QT * QTILE + QT * SUBQ + STAGES * 2 * KTILE) * 2 + (2 * STAGES + 9 * QT + ITEM_RING) * 8 + 64 + ITEM_RING * sizeof(Item);
}

// The q rows of a step as (64 columns of a head, heads, tokens): one box is half a Q tile, [128 / G tokens][G heads
// of one group][64], which is the tile's row order (token, head in group).
bool make_q_map(CUtensorMap* map, const void* q, long long q_row_stride, int Hq, long long n_tokens, int G) {
  auto fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)Hq, (cuuint64_t)n_tokens};
  cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)q_row_stride * 2};
  cuuint32_t box[3] = {64u, (cuuint32_t)G, (cuuint32_t)(ROWS / G)};
  cuuint32_t elem[3] = {1, 1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
}  // namespace
// Attention of the requests with at least `min_q_long` new tokens; the others are skipped (the split-key kernel
// serves them).  head_dim must be 128 and page_size one of 8 / 16 / 32 / 64; n_pages: pages of this cache layer;
// n_tokens: rows of q; work: two ints on the device, zero before the first launch and left zero by every launch
// that runs to its end.  Returns cudaErrorInvalidValue for what it cannot do, so the caller can fall back.
BSPEC_API int bspec_attention_prefill_tc(const void* q, long long q_row_stride, void* out, int* status,
                                         long long n_pages, const void* cache, const int* qo_indptr,
                                         const int* positions, const int* kv_indptr, const int* kv_indices,
                                         int n_entries, long long n_tokens, int max_q_len, int Hq, int Hkv, int hd,
                                         int page_size, float scale, int window, int min_q_long, int* work,
                                         cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return 0;
  if (hd != HD || Hq % Hkv != 0 || page_size % 8 != 0 || KT % page_size != 0 || status == nullptr || n_pages <= 0 ||
      n_tokens <= 0 || work == nullptr)
    return (int)cudaErrorInvalidValue;
  CUtensorMap kv_map, q_map;
  if (!make_map_2d_bf16(&kv_map, cache, n_pages * 2 * Hkv * page_size, HD, page_size, 64)) return (int)cudaErrorInvalidValue;
  const int G = Hq / Hkv;
  // Q through TMA when a tile's 128 rows are whole tokens (G divides 128) and the rows are 16-byte aligned;
  // otherwise the softmax threads copy their rows
  int q_by_tma = (ROWS % G == 0) && (q_row_stride % 8 == 0) && (((uintptr_t)q & 15) == 0);
  if (q_by_tma && !make_q_map(&q_map, q, q_row_stride, Hq, n_tokens, G)) q_by_tma = 0;
  if (!q_by_tma) q_map = kv_map;                                 // not read
  static bool attr_set_dev[bspec::kMaxDevices] = {};            // per device
  bool& attr_set = attr_set_dev[bspec::current_device()];
  if (!attr_set) {
    const cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)smem_bytes());
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const long long blocks = ((long long)max_q_len * G + QT * ROWS - 1) / (QT * ROWS);
  const long long n_items = blocks * Hkv * n_entries;
  if (n_items > (1ll << 30)) return (int)cudaErrorInvalidValue;
  const int grid = (int)(n_items < bspec::sm_count() ? n_items : bspec::sm_count());
  BSPEC_LAUNCH((attn_prefill_tc_kernel), dim3(grid), THREADS, smem_bytes(), stream, kv_map, q_map,
               (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, status, qo_indptr, positions, kv_indptr,
               kv_indices, Hq, Hkv, n_entries, (int)n_items, page_size, scale * 1.4426950408889634f, window, min_q_long,
               q_by_tma, work);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_attention_tcgen05)
