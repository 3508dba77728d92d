// bfloat16 matrix product for decode-sized steps (at most 128 tokens) on the 5th-generation tensor cores:
//   C[M, N] = X[M, K] * W[N, K]^T,   M <= 128,   weights on the accumulator's rows.
//
// Such a step is bound by reading W once, so every SM should stream the same number of weight bytes without
// pause.  The work is the sequence of (128-row tile of W, 64-wide K block) units, tile by tile; CTA b of G takes
// the units [b U / G, (b + 1) U / G) whatever the tile count is, and walks them without leaving the kernel:
//   warp 0   one thread issues the TMA loads of every unit (W block 128 x 64, X block bn x 64) into a ring of
//            shared-memory stages; the first stages' W blocks are fetched before the wait on the kernel before;
//   warp 1   one thread issues tcgen05.mma (128 x bn x 16, four per unit) into one of TWO accumulators in tensor
//            memory, so that the next tile's products start while the last tile's accumulator is drained;
//   warps 2-5 read an accumulator back (tcgen05.ld) and either finish the tile (it lay inside this CTA's units:
//            convert, optionally silu(gate) * up, store) or leave a float32 partial tile in scratch.
// Only the first and the last tile of a CTA can be shared with other CTAs.  Their partial tiles are announced
// after all of the CTA's units (one fence, one atomic per tile); each CTA that shares a tile then waits (bounded)
// until all of the tile's parts are announced and finishes its own share of the tile's tokens, adding the parts
// in their order.
//
// Every wait on an mbarrier is bounded: when it runs out the CTA records a code in `status`, stops issuing work,
// gives its tensor memory back and returns.
#include "common.cuh"
#include "tma.cuh"
#include "umma.cuh"

using namespace bspec;

namespace {

constexpr int BK = 64;                 // K elements per unit (one 128-byte swizzle span of bf16)
constexpr int TM = UMMA_M;             // rows of W per tile
constexpr int STREAM_THREADS = 192;
constexpr int MAX_PARTS = 32;          // CTAs that may share one tile

struct StreamParams {
  void* C;               // [M, N] (glu: [M, N / 2]) bf16 or f32
  float* scratch;        // [ctas][2][bn][128] partial tiles: slot 0 a CTA's first tile, slot 1 its last
  int* counters;         // [tiles][2] parts announced, shares finished: zero before the first launch, left zero
  int* status;           // 0, or the first error code
  int M, N, K;
  int out_f32;
  int glu;               // rows of W in groups of 128 = 64 gate rows + their 64 up rows; C = silu(gate) * up
  int bn;                // accumulator columns: M rounded up to 16
  int stages;
  int tiles, kb_total;
  int ctas;              // G: the grid
};

struct Cut {
  long long units;
  int ctas, kb_total;
  __device__ __forceinline__ long long start_of(int b) const { return (long long)b * units / ctas; }
  __device__ __forceinline__ int cta_of(long long u) const { return (int)(((u + 1) * ctas - 1) / units); }
};

// The piece of CTA b's units that begins at unit u: tile, K blocks [k0, k1), and how the tile is shared.
struct Segment {
  int tile, k0, k1, part, n_parts;
};
__device__ __forceinline__ Segment segment_at(const Cut& cut, long long u, long long end, int b) {
  Segment s;
  s.tile = (int)(u / cut.kb_total);
  s.k0 = (int)(u - (long long)s.tile * cut.kb_total);
  s.k1 = (int)min((long long)cut.kb_total, s.k0 + (end - u));
  const int first = cut.cta_of((long long)s.tile * cut.kb_total);
  s.n_parts = cut.cta_of((long long)(s.tile + 1) * cut.kb_total - 1) - first + 1;
  s.part = b - first;
  return s;
}

__device__ __forceinline__ void store_out(void* C, int out_f32, size_t idx, float v) {
  if (out_f32) reinterpret_cast<float*>(C)[idx] = v;
  else reinterpret_cast<__nv_bfloat16*>(C)[idx] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float silu(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ void bar_epilogue() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

__global__ void __launch_bounds__(STREAM_THREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   StreamParams p) {
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_dyn + 1023) & ~(uintptr_t)1023);
  const int a_bytes = TM * BK * 2, b_bytes = p.bn * BK * 2;
  const int stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)p.stages * stage_bytes);
  uint64_t* empty = full + p.stages;
  uint64_t* acc_full = empty + p.stages;                       // [2]
  uint64_t* acc_empty = acc_full + 2;                          // [2]
  float* swap_up = reinterpret_cast<float*>(acc_empty + 2);    // [2][16][64] up rows on their way to the gate rows
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(swap_up + 2 * 16 * 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const unsigned long long t_trace = bspec::g_trace_buf != nullptr ? bspec::global_timer() : 0ull;
  bspec::pdl_launch_dependents();           // the next kernel may start its own prologue and weight prefetch
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x;
  Cut cut;
  cut.units = (long long)p.tiles * p.kb_total;
  cut.ctas = p.ctas;
  cut.kb_total = p.kb_total;
  const long long u_begin = cut.start_of(b), u_end = cut.start_of(b + 1);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < 2 * p.bn) tmem_cols <<= 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full + i, 1);
      mbar_init(acc_empty + i, 4);          // one arrival per epilogue warp
    }
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
      // The weights do not depend on the kernel before this one: fetch them for the first stages at once, and
      // only then wait for that kernel to finish before touching the activations it wrote.
      const int n_units = (int)(u_end - u_begin);
      const int pre = min(n_units, p.stages);
      for (int i = 0; i < pre; ++i) {
        const long long u = u_begin + i;
        const int tile = (int)(u / p.kb_total), kb = (int)(u - (long long)tile * p.kb_total);
        mbar_expect_tx(full + i, (uint32_t)(a_bytes + b_bytes));
        tma_load_2d(smem + (size_t)i * stage_bytes, &map_w, full + i, kb * BK, tile * TM);
      }
      bspec::pdl_wait();
      bspec::trace_record(20, t_trace);
      for (int i = 0; i < pre; ++i) {
        const long long u = u_begin + i;
        const int tile = (int)(u / p.kb_total), kb = (int)(u - (long long)tile * p.kb_total);
        tma_load_2d(smem + (size_t)i * stage_bytes + a_bytes, &map_x, full + i, kb * BK, 0);
      }
      int armed = pre;
      for (int i = pre; i < n_units; ++i) {
        const int s = i % p.stages;
        const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
        if (!mbar_wait(empty + s, ph ^ 1u, abort_flag, p.status, 41)) break;
        const long long u = u_begin + i;
        const int tile = (int)(u / p.kb_total), kb = (int)(u - (long long)tile * p.kb_total);
        unsigned char* dst = smem + (size_t)s * stage_bytes;
        mbar_expect_tx(full + s, (uint32_t)(a_bytes + b_bytes));
        tma_load_2d(dst, &map_w, full + s, kb * BK, tile * TM);
        tma_load_2d(dst + a_bytes, &map_x, full + s, kb * BK, 0);
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
      int i = 0, seg_no = 0;
      for (long long u = u_begin; u < u_end && ok; ++seg_no) {
        const Segment sg = segment_at(cut, u, u_end, b);
        u += sg.k1 - sg.k0;
        const int buf = seg_no & 1;
        // the accumulator is free once the epilogue has drained its use before the last one
        ok = mbar_wait(acc_empty + buf, (((uint32_t)seg_no >> 1) & 1u) ^ 1u, abort_flag, p.status, 42);
        if (!ok) break;
        tc_fence_after();
        const uint32_t acc = tmem_base + (uint32_t)(buf * p.bn);
        for (int kb = sg.k0; kb < sg.k1 && ok; ++kb, ++i) {
          const int s = i % p.stages;
          const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
          ok = mbar_wait(full + s, ph, abort_flag, p.status, 43);
          if (!ok) break;
          tc_fence_after();
          unsigned char* a_src = smem + (size_t)s * stage_bytes;
          const uint64_t adesc = smem_desc(a_src), bdesc = smem_desc(a_src + a_bytes);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k)       // 16 bf16 = 32 bytes = 2 descriptor address units per step
            tc_mma(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb > sg.k0 || k > 0) ? 1u : 0u);
          tc_commit(empty + s);                    // the stage is free once these MMAs have read it
        }
        if (ok) tc_commit(acc_full + buf);         // the accumulator is complete once all MMAs are done
      }
    }
  } else {
    // epilogue warps: TMEM lanes 32 * (warp % 4) .. + 31  <->  rows of the tile
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int n_out = p.glu ? p.N / 2 : p.N;
    int n_pending = 0, pend_tile[2], pend_parts[2], pend_part[2];
    bool ok = true, waited = false;
    int seg_no = 0;
    for (long long u = u_begin; u < u_end && ok; ++seg_no) {
      const Segment sg = segment_at(cut, u, u_end, b);
      u += sg.k1 - sg.k0;
      const int buf = seg_no & 1;
      ok = mbar_wait(acc_full + buf, ((uint32_t)seg_no >> 1) & 1u, abort_flag, p.status, 44);
      if (!ok) break;
      tc_fence_after();
      if (!waited) {
        bspec::pdl_wait();                               // C and the scratch may still be read by the kernel before
        waited = true;
      }
      const uint32_t acc = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(buf * p.bn);
      if (sg.n_parts > 1) {
        // a float32 partial tile, [token][row]: slot 0 if this is the CTA's first tile, else slot 1
        float* dst = p.scratch + ((size_t)b * 2 + (seg_no == 0 ? 0 : 1)) * p.bn * TM + row;
        for (int c0 = 0; c0 < p.bn; c0 += 16) {
          uint32_t v[16];
          tc_ld16(acc + (uint32_t)c0, v);
          tc_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (c0 + j < p.M) dst[(size_t)(c0 + j) * TM] = __uint_as_float(v[j]);
        }
        if (n_pending < 2) {
          pend_tile[n_pending] = sg.tile;
          pend_parts[n_pending] = sg.n_parts;
          pend_part[n_pending] = sg.part;
          ++n_pending;
        }
      } else if (!p.glu) {
        // consecutive lanes write consecutive outputs of one token
        const int ra = sg.tile * TM + row;
        for (int c0 = 0; c0 < p.bn; c0 += 16) {
          uint32_t v[16];
          tc_ld16(acc + (uint32_t)c0, v);
          tc_wait_ld();
          if (ra < p.N) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < p.M) store_out(p.C, p.out_f32, (size_t)(c0 + j) * p.N + ra, __uint_as_float(v[j]));
          }
        }
      } else {
        // rows 0..63 are gate rows, rows 64..127 their up rows: the up values cross over through shared memory,
        // 16 tokens at a time, two buffers so that one barrier per step is enough
        const int ra = sg.tile * 64 + (row & 63);
        int flip = 0;
        for (int c0 = 0; c0 < p.bn; c0 += 16, flip ^= 1) {
          uint32_t v[16];
          tc_ld16(acc + (uint32_t)c0, v);
          tc_wait_ld();
          float* sw = swap_up + flip * 16 * 64;
          if (row >= 64) {
#pragma unroll
            for (int j = 0; j < 16; ++j) sw[j * 64 + (row - 64)] = __uint_as_float(v[j]);
          }
          bar_epilogue();
          if (row < 64 && ra < n_out) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (c0 + j < p.M)
                store_out(p.C, p.out_f32, (size_t)(c0 + j) * n_out + ra, silu(__uint_as_float(v[j])) * sw[j * 64 + row]);
          }
        }
        bar_epilogue();                          // the buffers are free for the next tile
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(acc_empty + buf);
    }
    if (threadIdx.x == 64) bspec::trace_mark(21, t_trace);      // every accumulator of this CTA drained
    // ---- tiles shared with other CTAs.  Every CTA first announces its parts (after one fence); then, for each
    // of its one or two shared tiles (two: half of the threads each, side by side), it waits until all parts of
    // the tile are announced and adds up ITS share of the tile (the part-th of n_parts equal runs of the tile's
    // values) over all parts in their order.  A CTA announces before it waits and its units never depend on
    // another CTA, so the waits end; they are bounded all the same.  The last CTA to finish its share resets the
    // tile's two counters.
    bar_epilogue();
    if (ok && !*abort_flag && n_pending > 0) {
      const int t128 = threadIdx.x - 64;
      __threadfence();
      bar_epilogue();
      if (t128 < n_pending) atomicAdd(&p.counters[2 * pend_tile[t128]], 1);
      if (threadIdx.x == 64) bspec::trace_mark(22, t_trace);    // parts announced
      const int group = n_pending == 2 ? 64 : 128;              // threads that work on one tile
      const int i = n_pending == 2 ? t128 >> 6 : 0, tg = t128 & (group - 1);
      const int bar_id = n_pending == 2 ? 2 + i : 1;
      auto bar_group = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(group) : "memory"); };
      const int tile = pend_tile[i], n_parts = pend_parts[i], me = pend_part[i];
      if (tg == 0) {
        const volatile int* arrived = p.counters + 2 * tile;
        uint32_t spins = 0;
        while (*arrived < n_parts) {
          if (++spins > WAIT_LIMIT || *abort_flag) {
            *abort_flag = 1;
            atomicCAS(p.status, 0, 45);
            break;
          }
          if (spins > 64) __nanosleep(32);
        }
      }
      bar_group();
      if (!*abort_flag) {
        __threadfence();
        if (threadIdx.x == 64) bspec::trace_mark(23, t_trace);  // all parts of the tile announced
        const int first = cut.cta_of((long long)tile * p.kb_total);
        // Part s > 0 comes from a CTA whose units begin inside this tile: it is that CTA's first piece (slot 0).
        // Part 0 is its CTA's last piece (slot 1) unless that CTA's units begin exactly with this tile.
        const bool late0 = cut.start_of(first) < (long long)tile * p.kb_total;
        const size_t part_stride = (size_t)2 * p.bn * TM;            // floats between CTAs' slot 0
        const float* base = p.scratch + (size_t)first * part_stride;
        auto sum4 = [&](int tok, int r0) {          // rows r0 .. r0 + 3 of token tok over all parts, four loads in flight
          const float* src = base + (size_t)tok * TM + r0;
          float4 acc = __ldcg(reinterpret_cast<const float4*>(src + (late0 ? (size_t)p.bn * TM : 0)));
          int sp = 1;
          for (; sp + 4 <= n_parts; sp += 4) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) v[u] = __ldcg(reinterpret_cast<const float4*>(src + (size_t)(sp + u) * part_stride));
#pragma unroll
            for (int u = 0; u < 4; ++u) { acc.x += v[u].x; acc.y += v[u].y; acc.z += v[u].z; acc.w += v[u].w; }
          }
          for (; sp < n_parts; ++sp) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(src + (size_t)sp * part_stride));
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
          }
          return acc;
        };
        auto store4 = [&](int tok, int ra, float4 v) {
          const size_t idx = (size_t)tok * n_out + ra;
          if (ra + 4 <= n_out && (n_out & 3) == 0) {
            if (p.out_f32) {
              *reinterpret_cast<float4*>(reinterpret_cast<float*>(p.C) + idx) = v;
            } else {
              __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
              *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(p.C) + idx) =
                  make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
            }
          } else {
            const float e[4] = {v.x, v.y, v.z, v.w};
            for (int j = 0; j < 4; ++j)
              if (ra + j < n_out) store_out(p.C, p.out_f32, idx + j, e[j]);
          }
        };
        if (!p.glu) {
          // the tile as M x 32 groups of four rows; this part's run of them
          const int n = p.M * 32, lo = (int)((long long)me * n / n_parts), hi = (int)((long long)(me + 1) * n / n_parts);
          for (int k = lo + tg; k < hi; k += group) store4(k >> 5, tile * TM + 4 * (k & 31), sum4(k >> 5, 4 * (k & 31)));
        } else {
          // the tile as M x 16 groups of four gate rows with their up rows 64 further on
          const int n = p.M * 16, lo = (int)((long long)me * n / n_parts), hi = (int)((long long)(me + 1) * n / n_parts);
          for (int k = lo + tg; k < hi; k += group) {
            const int tok = k >> 4, r0 = 4 * (k & 15);
            const float4 gt = sum4(tok, r0), up = sum4(tok, 64 + r0);
            store4(tok, tile * 64 + r0, make_float4(silu(gt.x) * up.x, silu(gt.y) * up.y, silu(gt.z) * up.z, silu(gt.w) * up.w));
          }
        }
        bar_group();
        if (threadIdx.x == 64) bspec::trace_mark(24, t_trace);  // share of the tile stored
        if (tg == 0) {
          if (atomicAdd(&p.counters[2 * tile + 1], 1) == n_parts - 1) {
            p.counters[2 * tile] = 0;
            p.counters[2 * tile + 1] = 0;
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
  }
}

size_t stream_smem_bytes(int bn, int stages) {
  const int a_bytes = TM * BK * 2, b_bytes = bn * BK * 2;
  const int stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
  return 1024 + (size_t)stages * stage_bytes + (size_t)(2 * stages + 4) * 8 + 2 * 16 * 64 * 4 + 64;
}

int g_force_ctas_per_sm = 0;
}  // namespace

// For experiments: CTAs per SM of the grid (0: choose automatically).
BSPEC_API void bspec_gemm_stream_ctas_per_sm(int n) { g_force_ctas_per_sm = n; }

// Plan for a product of these sizes: writes {bn, stages, ctas, tiles} to plan[4] and returns the bytes of scratch
// the launch needs (float32 partial tiles), or -1 if the sizes are not supported (M > 128, K not a multiple of 8).
BSPEC_API long long bspec_gemm_stream_plan(int M, int N, int K, int sm_count, int* plan) {
  if (M <= 0 || M > 128 || N <= 0 || K <= 0 || K % 8 != 0) return -1;
  const int bn = (M + 15) / 16 * 16;
  const int kb_total = (K + BK - 1) / BK, tiles = (N + TM - 1) / TM;
  const long long units = (long long)tiles * kb_total;
  const int a_bytes = TM * BK * 2, b_bytes = bn * BK * 2;
  const int stage_bytes = a_bytes + ((b_bytes + 1023) & ~1023);
  // Two CTAs per SM of about 100 KB each leave room for the neighbouring kernels' CTAs (whose prologues then
  // overlap with this kernel's tail, and this kernel's weight prefetch with theirs); wide token tiles need the
  // whole SM for a ring that is deep enough.
  int per_sm = (100 * 1024) / stage_bytes >= 4 ? 2 : 1;
  if (g_force_ctas_per_sm > 0) per_sm = g_force_ctas_per_sm;
  int stages = ((per_sm >= 2 ? 100 : 200) * 1024) / stage_bytes;
  if (stages > 12) stages = 12;
  if (stages < 2) stages = 2;
  // at least 2 units per CTA, and so many that no tile is shared by more than MAX_PARTS CTAs
  long long least = (kb_total + MAX_PARTS - 3) / (MAX_PARTS - 2);
  if (least < 2) least = 2;
  long long ctas = (long long)sm_count * per_sm;
  if (ctas > units / least) ctas = units / least;
  if (ctas < 1) ctas = 1;
  if (stages > units / ctas + 1) stages = (int)(units / ctas + 1) < 2 ? 2 : (int)(units / ctas + 1);
  plan[0] = bn; plan[1] = stages; plan[2] = (int)ctas; plan[3] = tiles;
  return ctas * 2 * bn * TM * 4;
}

// C = X W^T for M <= 128 tokens.  scratch: as many bytes as bspec_gemm_stream_plan returns; counters: int32
// [2 * tiles], zero before the first launch and left zero by every launch; status: one int on the device, 0 unless a
// bounded wait ran out.  glu != 0: the rows of W come in groups of 128 (64 gate rows, then the 64 matching up
// rows; N a multiple of 128) and C is [M, N / 2] = silu(gate) * up.
BSPEC_API int bspec_gemm_stream(const void* X, const void* W, void* C, int M, int N, int K, int out_f32, int glu,
                                float* scratch, int* counters, int* status, int sm_count, cudaStream_t stream) {
  int plan[4];
  if (bspec_gemm_stream_plan(M, N, K, sm_count, plan) < 0) return (int)cudaErrorInvalidValue;
  if (glu && (N % 128 != 0)) return (int)cudaErrorInvalidValue;
  StreamParams p;
  p.C = C; p.scratch = scratch; p.counters = counters; p.status = status;
  p.M = M; p.N = N; p.K = K; p.out_f32 = out_f32; p.glu = glu ? 1 : 0;
  p.bn = plan[0]; p.stages = plan[1]; p.ctas = plan[2]; p.tiles = plan[3];
  p.kb_total = (K + BK - 1) / BK;
  CUtensorMap map_w, map_x;
  if (!make_map_2d_bf16(&map_w, W, N, K, TM, BK) || !make_map_2d_bf16(&map_x, X, M, K, p.bn, BK))
    return (int)cudaErrorInvalidValue;
  const size_t smem = stream_smem_bytes(p.bn, p.stages);
  static size_t smem_set_dev[bspec::kMaxDevices] = {};          // per device
  size_t& smem_set = smem_set_dev[bspec::current_device()];
  if (smem > smem_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    cudaFuncSetAttribute(gemm_stream_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    smem_set = smem;
  }
  BSPEC_LAUNCH((gemm_stream_kernel), dim3(p.ctas), STREAM_THREADS, smem, stream, map_w, map_x, p);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_gemm_stream)
