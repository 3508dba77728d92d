// bfloat16 matrix product on the 5th-generation tensor cores of sm_100a:
//   C[M, N] = X[M, K] * W[N, K]^T      (X, W row-major with K contiguous; C bfloat16 or float32)
//
// One CTA computes one 128 x BN accumulator tile held in tensor memory (TMEM):
//   warp 0   one elected thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of the two operand
//            tiles of every 64-wide K block into a ring of shared-memory stages, signalled by mbarriers;
//   warp 1   allocates TMEM; one elected thread issues tcgen05.mma (kind::f16, 128 x BN x 16) four times per
//            stage straight from shared memory and releases the stage with tcgen05.commit;
//   warps 2-5 read the accumulator back with tcgen05.ld (each warp its own 32 TMEM lanes) and store C.
//
// Two arrangements share the kernel:
//   tokens on the accumulator's rows   (M large):  rows = 128 tokens, columns = BN outputs.
//   weights on the accumulator's rows  (M small):  rows = 128 outputs, columns = BN >= M tokens (rows of X past M
//            are zero-filled by TMA), so a decode step streams every weight once at full tile efficiency.  K may
//            be cut into `splits` <= 8 slices run by the CTAs of one thread-block cluster; each CTA leaves its
//            partial tile in its own shared memory and, after a cluster barrier, adds up its share of the tokens
//            over all slices, in slice order, reading the peers through distributed shared memory.
//
// Epilogues of the weights-on-rows arrangement: plain store; silu(gate) * up for the fused gate/up projection; and,
// for the fused q/k/v projection of an attention layer whose head size is the tile's 128 rows, rotary encoding of
// the q and k heads (angle in float64, rotation in float32, on the float32 accumulators) with k and v written
// straight into their cache pages: one kernel instead of three, and one rounding to bfloat16 instead of two.
//
// Every wait on an mbarrier is bounded: when it runs out the CTA records a code in `status`, stops issuing work,
// gives its TMEM back and returns.
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

using namespace bspec;

namespace {

constexpr int BK = 64;                 // K elements per stage (one 128-byte swizzle span of bf16)
constexpr int TM = 128;                // accumulator rows (UMMA M)
constexpr int GEMM_THREADS = 192;

struct GemmParams {
  void* C;               // [M, N] bf16 or f32
  int* status;           // 0, or the first error code
  int M, N, K;
  int out_f32;
  int swap;              // 1: weights on the accumulator rows
  int bn;                // accumulator columns
  int splits;
  int kblocks_per_split;
  int stages;
  int glu;               // rows of W come in groups of 16 = 8 gate rows + their 8 up rows; C[M, N/2] = silu(gate) * up
  int prefetch_kb;       // K blocks of weights (beyond the stages) to pull into the L2 before waiting on the predecessor
  // fused q/k/v projection (rope_freq != nullptr): tile t of W is head t (q heads, then k heads, then v heads)
  const float* rope_freq;    // [2][64] frequencies as two floats each (see elementwise.cu, rope_sincos)
  const int* positions;      // [M]
  const int* tok_entry;      // [M]
  const int* kv_indptr;      // block tables of the step, CSR
  const int* kv_indices;
  __nv_bfloat16* cache;      // this layer's pages [page][k|v][Hkv][page_size][128]
  int Hq, Hkv, page_size, interleaved, write_kv;
  long long n_pages;         // pages of the cache layer (read by the checked build only)
};

// cos and sin of position * frequency j, the angle formed and reduced to [-pi, pi] in float64 (as elementwise.cu).
__device__ __forceinline__ void rope_sincos64(int pos, const float* __restrict__ freq, int j, float* s, float* c) {
  const double f = (double)freq[j] + (double)freq[64 + j];
  double a = (double)pos * f;
  a -= 6.283185307179586476925286766559 * rint(a * 0.15915494309189533576888376337251);
  sincosf((float)a, s, c);
}

__device__ __forceinline__ void store_out(void* C, int out_f32, size_t idx, float v) {
  if (out_f32) reinterpret_cast<float*>(C)[idx] = v;
  else reinterpret_cast<__nv_bfloat16*>(C)[idx] = __float2bfloat16_rn(v);
}

__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, GemmParams p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int a_bytes = TM * BK * 2, b_bytes = p.bn * BK * 2;
  const int stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * stage_bytes);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* part = reinterpret_cast<float*>(smem);      // [bn][128] partial tile of this K slice (reuses the stages)

  const unsigned long long t_trace = bspec::g_trace_buf != nullptr ? bspec::global_timer() : 0ull;
  bspec::pdl_launch_dependents();           // the next kernel may start its own prologue and weight prefetch
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile_a = blockIdx.x;            // 128-row tile of the operand on the accumulator rows
  const int tile_b = blockIdx.y;            // bn-row tile of the other operand
  const int split = blockIdx.z;
  const int kb_total = (p.K + BK - 1) / BK;
  const int kb0 = split * p.kblocks_per_split;
  const int nkb = min(p.kblocks_per_split, kb_total - kb0);      // >= 1 by construction on the host
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < p.bn) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(s32(tmem_slot)), "r"(tmem_cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      int armed = 0;
      // The weights do not depend on the kernel before this one: fetch them for the first stages at once, and
      // only then wait for that kernel to finish before touching the activations it wrote.
      const int pre = min(nkb, p.stages);
      for (int i = 0; i < pre; ++i) {
        unsigned char* a_dst = smem + (size_t)i * stage_bytes;
        mbar_expect_tx(full + i, (uint32_t)(a_bytes + b_bytes));
        if (p.swap) tma_load_2d(a_dst, &map_a, full + i, (kb0 + i) * BK, tile_a * TM);
        else tma_load_2d(a_dst + a_bytes, &map_b, full + i, (kb0 + i) * BK, tile_b * p.bn);
      }
      const int pf_end = min(nkb, pre + p.prefetch_kb);
      for (int i = pre; i < pf_end; ++i) {
        if (p.swap) tma_prefetch_2d(&map_a, (kb0 + i) * BK, tile_a * TM);
        else tma_prefetch_2d(&map_b, (kb0 + i) * BK, tile_b * p.bn);
      }
      bspec::pdl_wait();
      bspec::trace_record(20, t_trace);
      for (int i = 0; i < pre; ++i) {
        unsigned char* a_dst = smem + (size_t)i * stage_bytes;
        if (p.swap) tma_load_2d(a_dst + a_bytes, &map_b, full + i, (kb0 + i) * BK, tile_b * p.bn);
        else tma_load_2d(a_dst, &map_a, full + i, (kb0 + i) * BK, tile_a * TM);
      }
      armed = pre;
      for (int i = pre; i < nkb; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        if (!mbar_wait(empty + s, ph ^ 1u, abort_flag, p.status, 1)) break;
        unsigned char* a_dst = smem + (size_t)s * stage_bytes;
        mbar_expect_tx(full + s, (uint32_t)(a_bytes + b_bytes));
        tma_load_2d(a_dst, &map_a, full + s, (kb0 + i) * BK, tile_a * TM);
        tma_load_2d(a_dst + a_bytes, &map_b, full + s, (kb0 + i) * BK, tile_b * p.bn);
        armed = i + 1;
      }
      if (*abort_flag) {
        // let copies that are still in flight land before the CTA's shared memory is given up
        for (int i = max(0, armed - p.stages); i < armed; ++i) {
          const int s = i % p.stages;
          const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
          for (uint32_t t = 0; t < (1u << 16) && !mbar_try_wait(full + s, ph); ++t) __nanosleep(32);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = instr_desc(p.bn);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        ok = mbar_wait(full + s, ph, abort_flag, p.status, 2);
        if (!ok) break;
        tc_fence_after();
        unsigned char* a_src = smem + (size_t)s * stage_bytes;
        const uint64_t adesc = smem_desc(a_src), bdesc = smem_desc(a_src + a_bytes);
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)       // 16 bf16 = 32 bytes = 2 descriptor address units per step
          tc_mma(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        tc_commit(empty + s);                    // the stage is free once these MMAs have read it
      }
      if (ok) tc_commit(acc_full);               // the accumulator is complete once all MMAs are done
    }
  } else {
    // epilogue warps: TMEM lanes 32*(warp%4) .. +31  <->  accumulator rows
    const int quad = warp & 3;
    const int row = quad * 32 + lane;                       // accumulator row of this thread
    const bool ok = mbar_wait(acc_full, 0, abort_flag, p.status, 3);
    tc_fence_after();
    if (threadIdx.x == 64) bspec::trace_mark(21, t_trace);      // accumulator complete
    bspec::pdl_wait();                                      // C may reuse memory the kernel before still reads
    if (ok) {
      const int ra = tile_a * TM + row;                     // global row of the operand on the accumulator rows
      for (int c0 = 0; c0 < p.bn; c0 += 16) {
        uint32_t v[16];
        tc_ld16(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
        tc_wait_ld();
        if (!p.swap && p.glu) {
          // rows = tokens, columns = outputs in groups of 8 gate + 8 up: this chunk of 16 holds 8 outputs whole
          const int n0 = tile_b * p.bn + c0;                         // gate column; output column n0 / 2
          if (ra < p.M) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (n0 + 8 + j < p.N) {
                const float gte = __uint_as_float(v[j]);
                store_out(p.C, p.out_f32, (size_t)ra * (p.N / 2) + (n0 >> 1) + j,
                          gte / (1.f + expf(-gte)) * __uint_as_float(v[8 + j]));
              }
          }
        } else if (!p.swap) {
          // rows = tokens (ra < M), columns = outputs
          if (ra < p.M) {
            const int n0 = tile_b * p.bn + c0;
            const size_t base = (size_t)ra * p.N + n0;
            if (!p.out_f32 && n0 + 16 <= p.N && (p.N % 8) == 0) {
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                w[j] = *reinterpret_cast<uint32_t*>(&h);
              }
              uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(p.C) + base);
              dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
              dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j)
                if (n0 + j < p.N) store_out(p.C, p.out_f32, base + j, __uint_as_float(v[j]));
            }
          }
        } else if (p.splits == 1 && !p.glu && p.rope_freq == nullptr) {
          // rows = outputs (ra < N), columns = tokens: consecutive lanes write consecutive outputs of one token
          if (ra < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int tok = tile_b * p.bn + c0 + j;
              if (tok < p.M) store_out(p.C, p.out_f32, (size_t)tok * p.N + ra, __uint_as_float(v[j]));
            }
          }
        } else {
          // every MMA has completed (acc_full), so the stages are no longer read: keep the partial tile there
#pragma unroll
          for (int j = 0; j < 16; ++j) part[(size_t)(c0 + j) * TM + row] = __uint_as_float(v[j]);
        }
      }
    }
  }
  if (p.swap && (p.splits > 1 || p.glu || p.rope_freq != nullptr)) {
    // join the K slices inside the cluster: CTA r adds tokens r, r + splits, ... over all slices in slice order
    tc_fence_before();
    __syncthreads();
    if (p.splits > 1)
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (threadIdx.x == 64) bspec::trace_mark(22, t_trace);      // partial tiles of the cluster visible
    if (warp >= 2 && !*abort_flag) {
      const int row = (warp & 3) * 32 + lane;
      // plain: this thread owns output row `row` of the tile.  glu: the threads of gate rows (row & 8 == 0) own that
      // row and the up row 8 further and produce output tile_a * 64 + (row / 16) * 8 + row % 8 of the N / 2 outputs.
      const bool active = p.glu ? (row & 8) == 0 : true;
      const int ra = p.glu ? tile_a * 64 + (row >> 4) * 8 + (row & 7) : tile_a * TM + row;
      const int n_out = p.glu ? p.N / 2 : p.N;
      if (active && ra < n_out) {
        // addresses of this thread's row(s) in every peer's partial tile
        uint32_t peer[8];
        const uint32_t mine = s32(part + row);
#pragma unroll
        for (int s = 0; s < 8; ++s)
          if (s < p.splits) asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer[s]) : "r"(mine), "r"(s));
        // four tokens at a time, all their loads in flight before the first add: a load from a peer's shared
        // memory takes some hundred cycles, and with 64 tokens on the tile a CTA has up to 32 of them to join
        for (int j0 = split; j0 < p.bn; j0 += 4 * p.splits) {
          float v[4][8], u[4][8];
          bool live[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const int j = j0 + t * p.splits;
            live[t] = j < p.bn && tile_b * p.bn + j < p.M;
            if (live[t]) {
              const uint32_t off = (uint32_t)j * TM * 4u;
#pragma unroll
              for (int s = 0; s < 8; ++s)
                if (s < p.splits) {
                  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v[t][s]) : "r"(peer[s] + off));
                  if (p.glu) asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(u[t][s]) : "r"(peer[s] + off + 32u));
                }
            }
          }
          float res[4];
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            float acc = 0.f, acc_u = 0.f;
            if (live[t]) {
#pragma unroll
              for (int s = 0; s < 8; ++s)
                if (s < p.splits) {                          // slice order
                  acc += v[t][s];
                  if (p.glu) acc_u += u[t][s];
                }
              if (p.glu) acc = acc / (1.f + expf(-acc)) * acc_u;
            }
            res[t] = acc;
          }
          if (p.rope_freq == nullptr) {
#pragma unroll
            for (int t = 0; t < 4; ++t)
              if (live[t])
                store_out(p.C, p.out_f32, (size_t)(tile_b * p.bn + j0 + t * p.splits) * n_out + ra, res[t]);
          } else {
            // This tile is one head (128 rows): thread `row` holds dim `row` of the head for up to four tokens
            // and needs its rotary partner's value, which another thread of this CTA holds.  All 128 threads of
            // the four epilogue warps get here (N is a multiple of 128), so they can meet at a named barrier.
            float* xchg = part + (size_t)p.bn * TM;                 // [4][128], behind the partial tile
            const int head = tile_a;
            const bool is_v = head >= p.Hq + p.Hkv;
#pragma unroll
            for (int t = 0; t < 4; ++t) xchg[t * TM + row] = res[t];
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int partner = p.interleaved ? (row ^ 1) : (row ^ 64);
            const bool first = p.interleaved ? ((row & 1) == 0) : (row < 64);
            const int fj = p.interleaved ? (row >> 1) : (row & 63);
#pragma unroll
            for (int t = 0; t < 4; ++t) {
              if (!live[t]) continue;
              const int tok = tile_b * p.bn + j0 + t * p.splits;
              const int pos = p.positions[tok];
              float val = res[t];
              if (!is_v) {
                float sn, cs;
                rope_sincos64(pos, p.rope_freq, fj, &sn, &cs);
                const float other = xchg[t * TM + partner];
                val = first ? res[t] * cs - other * sn : other * sn + res[t] * cs;
              }
              const __nv_bfloat16 b = __float2bfloat16_rn(val);
              if (head < p.Hq) {
                reinterpret_cast<__nv_bfloat16*>(p.C)[(size_t)tok * p.N + ra] = b;
              } else if (p.write_kv) {
                const int e = p.tok_entry[tok];
                if (!bspec::in_range(pos / p.page_size, p.kv_indptr[e + 1] - p.kv_indptr[e], 105)) continue;
                const long long page = p.kv_indices[p.kv_indptr[e] + pos / p.page_size];
                if (!bspec::in_range(page, p.n_pages, 106)) continue;
                const int kvh = is_v ? head - p.Hq - p.Hkv : head - p.Hq;
                const size_t at = (((size_t)page * 2 + (is_v ? 1 : 0)) * p.Hkv + kvh) * p.page_size * TM +
                                  (size_t)(pos % p.page_size) * TM + row;
                p.cache[at] = b;
              }
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");         // before the next four tokens reuse xchg
          }
        }
      }
    }
    if (threadIdx.x == 64) bspec::trace_mark(23, t_trace);      // joined and stored
    // nobody leaves while a peer may still read its shared memory
    if (p.splits > 1)
      asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (threadIdx.x == 64) bspec::trace_mark(24, t_trace);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

// ---------------------------------------------------------------------------------------------------- host side
size_t smem_bytes(int bn, int stages) {
  const int a_bytes = TM * BK * 2, b_bytes = bn * BK * 2;
  const int stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
  return 1024 + (size_t)stages * stage_bytes + (size_t)(2 * stages + 1) * 8 + 64;
}
}  // namespace

static int g_force_splits = 0;
// For experiments: force the number of K slices of the weights-on-rows arrangement (0: choose automatically).
BSPEC_API void bspec_gemm_tc_force_splits(int splits) { g_force_splits = splits > 8 ? 8 : splits; }

// Plan for a product of these sizes: writes {swap, bn, splits, stages, tiles} to plan[5]; returns 0, or -1 if the
// sizes are not supported (K not a multiple of 8).  `sm_count` is the number of SMs to fill.
BSPEC_API long long bspec_gemm_tc_plan(int M, int N, int K, int sm_count, int* plan) {
  if (K % 8 != 0 || M <= 0 || N <= 0 || K <= 0) return -1;
  const int kb_total = (K + BK - 1) / BK;
  int swap, bn, splits = 1;
  int smem_budget;
  if (M <= 128) {
    swap = 1;
    bn = 16;
    while (bn < M) bn <<= 1;
    const int tiles = (N + TM - 1) / TM;
    // Two CTAs share an SM: cut K into slices (the CTAs of one cluster, at most 8) so that the CTAs about fill
    // those slots, keeping at least 8 K blocks per slice.  Measured on B200: more, shorter slices lose more to the
    // per-CTA prologue and epilogue than they gain in balance.
    splits = (2 * sm_count) / tiles;
    if (splits < 1) splits = 1;
    if (splits > kb_total / 8) splits = kb_total / 8 > 0 ? kb_total / 8 : 1;
    if (splits > 8) splits = 8;
    while (splits & (splits - 1)) --splits;               // clusters of 1, 2, 4 or 8 schedule best (measured: 6 is slow)
    if (g_force_splits > 0) splits = g_force_splits < kb_total ? g_force_splits : kb_total;
    smem_budget = 108 * 1024;
  } else {
    swap = 0;
    bn = N >= 256 ? 256 : (N > 64 ? 128 : 64);
    smem_budget = 200 * 1024;
  }
  int per = (kb_total + splits - 1) / splits;
  splits = (kb_total + per - 1) / per;                   // no empty slice
  const int a_bytes = TM * BK * 2, b_bytes = bn * BK * 2;
  const int stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
  int stages = smem_budget / stage_bytes;
  if (stages > 8) stages = 8;
  if (stages > per + 1) stages = per + 1;
  if (stages < 2) stages = 2;
  const int tiles_a = swap ? (N + TM - 1) / TM : (M + TM - 1) / TM;
  const int tiles_b = swap ? (M + bn - 1) / bn : (N + bn - 1) / bn;
  plan[0] = swap; plan[1] = bn; plan[2] = splits; plan[3] = stages; plan[4] = tiles_a * tiles_b;
  return 0;
}

struct RopeEpilogue {
  const float* freq;
  const int* positions;
  const int* tok_entry;
  const int* kv_indptr;
  const int* kv_indices;
  void* cache;
  int Hq, Hkv, page_size, interleaved, write_kv;
  long long n_pages;
};

static int launch_gemm(const void* X, const void* W, void* C, int M, int N, int K, int out_f32, int glu, int* status,
                       int sm_count, const RopeEpilogue* rope, cudaStream_t stream) {
  int plan[5];
  if (bspec_gemm_tc_plan(M, N, K, sm_count, plan) < 0) return (int)cudaErrorInvalidValue;
  if (glu && (N % 16 != 0)) return (int)cudaErrorInvalidValue;
  GemmParams p;
  p.C = C; p.status = status;
  p.M = M; p.N = N; p.K = K; p.out_f32 = out_f32; p.glu = glu ? 1 : 0;
  p.swap = plan[0]; p.bn = plan[1]; p.splits = plan[2]; p.stages = plan[3];
  p.rope_freq = nullptr; p.positions = p.tok_entry = p.kv_indptr = p.kv_indices = nullptr; p.cache = nullptr;
  p.Hq = p.Hkv = p.page_size = p.interleaved = p.write_kv = 0;
  p.n_pages = 0;
  if (rope != nullptr) {
    // one 128-row tile per head, on the weights-on-rows arrangement, bfloat16 out, room behind the partial tile
    const int stage_bytes = TM * BK * 2 + ((p.bn * BK * 2 + 1023) & ~1023);
    if (!p.swap || glu || out_f32 || N != (rope->Hq + 2 * rope->Hkv) * TM || rope->page_size < 1 ||
        (size_t)(p.bn + 4) * TM * 4 > (size_t)p.stages * stage_bytes)
      return (int)cudaErrorInvalidValue;
    p.rope_freq = rope->freq; p.positions = rope->positions; p.tok_entry = rope->tok_entry;
    p.kv_indptr = rope->kv_indptr; p.kv_indices = rope->kv_indices; p.cache = (__nv_bfloat16*)rope->cache;
    p.Hq = rope->Hq; p.Hkv = rope->Hkv; p.page_size = rope->page_size; p.interleaved = rope->interleaved;
    p.write_kv = rope->write_kv;
    p.n_pages = rope->n_pages;
  }
  const int kb_total = (K + BK - 1) / BK;
  p.kblocks_per_split = (kb_total + p.splits - 1) / p.splits;
  {
    // weights this launch may park in the L2 ahead of time: at most 48 MB (the L2 has 126 MB)
    const long long ctas = (long long)plan[4] * p.splits;
    const long long per_kb = ctas * (p.swap ? TM : p.bn) * BK * 2;
    long long pf = per_kb > 0 ? (48ll << 20) / per_kb : 0;
    if (pf > p.kblocks_per_split) pf = p.kblocks_per_split;
    p.prefetch_kb = bspec::pdl_enabled() ? (int)pf : 0;
  }
  CUtensorMap map_a, map_b;
  const void* a_ptr = p.swap ? W : X;
  const void* b_ptr = p.swap ? X : W;
  const int a_rows = p.swap ? N : M, b_rows = p.swap ? M : N;
  if (!make_map_2d_bf16(&map_a, a_ptr, a_rows, K, TM, BK) || !make_map_2d_bf16(&map_b, b_ptr, b_rows, K, p.bn, BK))
    return (int)cudaErrorInvalidValue;
  const size_t smem = smem_bytes(p.bn, p.stages);
  static size_t smem_set_dev[bspec::kMaxDevices] = {};          // per device
  size_t& smem_set = smem_set_dev[bspec::current_device()];
  if (smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    smem_set = smem;
  }
  dim3 grid((a_rows + TM - 1) / TM, (b_rows + p.bn - 1) / p.bn, p.splits);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(GEMM_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = p.splits;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = bspec::pdl_enabled() ? 2 : 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tc_kernel, map_a, map_b, p);
  if (e != cudaSuccess) return (int)e;
  return BSPEC_LAUNCH_CHECK();
}

// C = X W^T.  `status`: one int on the device, 0 unless a bounded wait ran out.
// glu != 0: the rows of W come in groups of 16 (8 gate rows, then the 8 matching up rows; N a multiple of 16) and
// C is [M, N/2] = silu(gate) * up.
BSPEC_API int bspec_gemm_tc(const void* X, const void* W, void* C, int M, int N, int K, int out_f32, int glu,
                            int* status, int sm_count, cudaStream_t stream) {
  return launch_gemm(X, W, C, M, N, K, out_f32, glu, status, sm_count, nullptr, stream);
}

// The fused q/k/v projection of an attention layer with head size 128 for a step of at most 128 tokens:
// W = [Wq; Wk; Wv] with Hq + 2 Hkv heads of 128 rows, C [M, N] bfloat16.  The q heads are rotated and stored to C
// (the k and v columns of C are left untouched); the k heads are rotated and, with the v heads, written into the
// cache page of each token's position (`write_kv` 0: not written).  freq: [2][64] float (leading parts, then
// remainders, of the 64 frequencies); pairing (j, j + 64), or (2j, 2j + 1) with `interleaved`.
// Returns cudaErrorInvalidValue for sizes this epilogue does not take; nothing is launched then.
BSPEC_API int bspec_gemm_tc_qkv_rope(const void* X, const void* W, void* C, int M, int N, int K, int* status, int sm_count,
                                     const float* freq, const int* positions, const int* tok_entry,
                                     const int* kv_indptr, const int* kv_indices, void* cache, int Hq, int Hkv,
                                     int page_size, int interleaved, int write_kv, long long n_pages,
                                     cudaStream_t stream) {
  const RopeEpilogue rope = {freq, positions, tok_entry, kv_indptr, kv_indices, cache, Hq, Hkv, page_size,
                             interleaved, write_kv, n_pages};
  return launch_gemm(X, W, C, M, N, K, 0, 0, status, sm_count, &rope, stream);
}

// Switch programmatic dependent launch on (default) or off for every kernel of this library.
BSPEC_API void bspec_set_pdl(int on) { bspec::pdl_enabled() = on != 0; }

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_gemm_tcgen05)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_gemm_tcgen05)
