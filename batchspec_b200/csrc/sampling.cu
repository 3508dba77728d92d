// Next-token selection from float32 logits [rows, vocab]: argmax (temperature 0),
// and sampling from softmax(logits / T) restricted by top-k and/or top-p.
// Three small kernels: per-row thresholds, sliced arg-best, final pick.  Randomness is a counter-based hash of (seed, stream id,
// draw counter, token index): a row's draw does not depend on the batch it is in.
//
// Restriction, then Gumbel-max: token i is kept if it is among the top_k largest
// logits (ties at the k-th value are all kept) and, of those, if the probability
// mass of strictly larger logits is below top_p; the sample is
// argmax_i (logit_i / T - log(-log u_i)) over kept tokens, which is a draw from the
// renormalised distribution.
#include "common.cuh"
#include <math.h>
using namespace bspec;

namespace {
constexpr int THREADS = 1024;

__device__ __forceinline__ uint32_t order_key(float x) {   // monotone map float -> uint32
  uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z ^= z >> 31; z *= 0x9E3779B97F4A7C15ull;
  z ^= z >> 29; z *= 0xD6E8FEB86659FD93ull;
  z ^= z >> 32; z *= 0xCA5A826395121157ull;
  z ^= z >> 30;
  return z;
}

// uniform in (0, 1)
__device__ __forceinline__ float uniform01(uint64_t seed, uint64_t stream, uint64_t counter, uint32_t index) {
  uint64_t z = mix64(seed ^ mix64(stream + 0x632BE59BD9B4E019ull));
  z = mix64(z ^ mix64(counter * 0x9E3779B97F4A7C15ull + index));
  return ((float)(uint32_t)(z >> 40) + 0.5f) * (1.0f / 16777216.0f);
}

struct ArgBest { float v; int i; };

__device__ __forceinline__ ArgBest better(ArgBest a, ArgBest b) {   // larger value, then smaller index
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ ArgBest block_argmax(ArgBest x, ArgBest* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y{__shfl_xor_sync(0xffffffffu, x.v, o), __shfl_xor_sync(0xffffffffu, x.i, o)};
    x = better(x, y);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = x;
  __syncthreads();
  ArgBest t = lane < nw ? scratch[lane] : ArgBest{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y{__shfl_xor_sync(0xffffffffu, t.v, o), __shfl_xor_sync(0xffffffffu, t.i, o)};
    t = better(t, y);
  }
  return t;
}

__device__ int block_count(int v, int* iscratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) iscratch[warp] = v;
  __syncthreads();
  int t = lane < nw ? iscratch[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;
}

// Stage 1 (one block per row): the smallest ordered key a token must reach to stay in the top-k / top-p set;
// 0 (everything stays) for rows that are greedy or unrestricted, which leave at once.
//
// Three passes over the row.  (1) Its largest and smallest finite logit.  (2) A histogram over BINS equal steps of
// the logit's value: of counts between smallest and largest for top-k, of probability mass over the 22 T below
// the largest (below that a token's mass rounds to nothing) for top-p alone.  A scan from the top bin finds the bin
// in which the k-th token lies (in which the mass reaches top_p).  (3) The tokens of that bin (with top-k: of that bin
// and all above it, which are then all that top-p has to weigh) go to a list in shared memory, where the exact key is
// found by comparing every listed token with every other.  Mass is summed in 64-bit fixed point (2^-30 of the largest
// token's mass), so a sum does not depend on the order of its terms, and the threshold is the same in every run and
// batch.  Rows whose list would not fit (k above LIST, thousands of equal logits) are bisected on the key bits
// instead, one pass per bit.
using u64 = unsigned long long;
constexpr int BINS = 4096;
constexpr int LIST = 2048;
static_assert(BINS % THREADS == 0, "each thread scans BINS / THREADS bins");

__device__ __forceinline__ uint32_t mass_of(float x, float mx, float invT) {   // at most 2^30
  return (uint32_t)(expf((x - mx) * invT) * 1073741824.f + 0.5f);
}

__device__ __forceinline__ int bin_of(float x, float lo, float inv_step) {   // monotone in x; NaN and -inf to bin 0
  return (int)fminf(fmaxf((x - lo) * inv_step, 0.f), (float)(BINS - 1));
}

template <class F>
__device__ __forceinline__ void for_each_logit(const float* __restrict__ row, int vocab, F f) {
  if ((vocab & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
    const float4* r4 = reinterpret_cast<const float4*>(row);
    for (int i = threadIdx.x; i < (vocab >> 2); i += blockDim.x) {
      const float4 v = r4[i];
      f(v.x); f(v.y); f(v.z); f(v.w);
    }
  } else {
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) f(row[i]);
  }
}

__device__ u64 block_sum_u64(u64 v, u64* wsum) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  __syncthreads();
  if (lane == 0) wsum[warp] = v;
  __syncthreads();
  u64 t = lane < nw ? wsum[lane] : 0;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  __syncthreads();
  return t;
}

// Every thread gets the largest bin d with sum(hist[d..BINS)) >= need, and what of need is left for that bin.
// need is at least 1 and at most the histogram's total.  WIDE: a bin is hi[b] * 2^32 + lo[b].
template <bool WIDE>
__device__ void select_bin(const uint32_t* lo, const uint32_t* hi, u64 need, u64* wsum, u64* sel, int& d, u64& rem) {
  constexpr int PER = BINS / THREADS;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  u64 h[PER];
  u64 local = 0;
#pragma unroll
  for (int j = 0; j < PER; ++j) {
    const int b = BINS - 1 - (t * PER + j);
    h[j] = WIDE ? (((u64)hi[b] << 32) | lo[b]) : (u64)lo[b];
    local += h[j];
  }
  u64 incl = local;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const u64 y = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += y;
  }
  if (lane == 31) wsum[warp] = incl;
  __syncthreads();
  for (int w = 0; w < warp; ++w) incl += wsum[w];
  u64 run = incl - local;
  if (run < need && need <= incl) {
#pragma unroll
    for (int j = 0; j < PER; ++j) {
      if (run < need && need <= run + h[j]) { sel[0] = (u64)(BINS - 1 - (t * PER + j)); sel[1] = need - run; }
      run += h[j];
    }
  }
  __syncthreads();
  d = (int)sel[0];
  rem = sel[1];
  __syncthreads();
}

__device__ __forceinline__ u64 share_of(float p, u64 z) {
  const u64 need = (u64)((double)p * (double)z);
  return need < 1 ? 1 : (need > z ? z : need);
}

struct ThresholdShared {
  uint32_t lo[BINS];        // counts, or the low words of the mass; then the list's keys
  u64 wide[BINS / 2];       // the high words of the mass, as uint32[BINS]; then the list's masses
  u64 wsum[32];
  u64 sel[2];
  float fscratch[64];
  int iscratch[32];
  int n_list;
  uint32_t best;
};

// False (for the whole block) if the row does not fit the lists; the threshold is then not written.
__device__ bool threshold_binned(const float* __restrict__ row, int vocab, float mx, float mn, float T, int k, float p,
                                 bool use_k, bool use_p, ThresholdShared& sh, uint32_t& th) {
  const float invT = 1.f / T;
  uint32_t* hi = reinterpret_cast<uint32_t*>(sh.wide);
  uint32_t* lkey = sh.lo;
  u64* lmass = sh.wide;
  const float lo_v = use_k ? mn : mx - 22.f * T;
  const float inv_step = (float)BINS / (mx - lo_v);
  if (!(inv_step < INFINITY) || !(inv_step > 0.f)) return false;
  for (int i = threadIdx.x; i < BINS; i += blockDim.x) { sh.lo[i] = 0; hi[i] = 0; }
  if (threadIdx.x == 0) { sh.n_list = 0; sh.best = 0xffffffffu; }
  __syncthreads();
  int d;
  u64 need = 0, above = 0;   // top-p alone: the mass to reach, and the mass of the bins above d
  if (use_k) {
    for_each_logit(row, vocab, [&](float x) { atomicAdd(&sh.lo[bin_of(x, lo_v, inv_step)], 1u); });
    __syncthreads();
    u64 rem;
    select_bin<false>(sh.lo, nullptr, (u64)k, sh.wsum, sh.sel, d, rem);
    const u64 n = (u64)k - rem + sh.lo[d];
    __syncthreads();
    if (n > LIST) return false;
  } else {
    for_each_logit(row, vocab, [&](float x) {
      const uint32_t w = mass_of(x, mx, invT);
      if (w) {
        const int b = bin_of(x, lo_v, inv_step);
        const uint32_t old = atomicAdd(&sh.lo[b], w);
        if (old + w < old) atomicAdd(&hi[b], 1u);
      }
    });
    __syncthreads();
    u64 z = 0;
    for (int i = threadIdx.x; i < BINS; i += blockDim.x) z += ((u64)hi[i] << 32) | sh.lo[i];
    z = block_sum_u64(z, sh.wsum);
    need = share_of(p, z);
    u64 rem;
    select_bin<true>(sh.lo, hi, need, sh.wsum, sh.sel, d, rem);
    above = need - rem;
  }
  // the list: with top-k every token from bin d up, else the tokens of bin d that have mass
  for_each_logit(row, vocab, [&](float x) {
    const int b = bin_of(x, lo_v, inv_step);
    if (use_k ? b < d : b != d) return;
    const uint32_t w = use_p ? mass_of(x, mx, invT) : 0u;
    if (!use_k && w == 0) return;
    const int slot = atomicAdd(&sh.n_list, 1);
    if (slot < LIST) { lkey[slot] = order_key(x); lmass[slot] = w; }
  });
  __syncthreads();
  const int n = sh.n_list;
  if (n > LIST) return false;
  uint32_t kth = 0;
  if (use_k) {   // the k-th largest key: the smallest listed key with fewer than k keys above it
    for (int e = threadIdx.x; e < n; e += blockDim.x) {
      const uint32_t key = lkey[e];
      int gt = 0;
      for (int j = 0; j < n; ++j) gt += lkey[j] > key;
      if (gt < k) atomicMin(&sh.best, key);
    }
    __syncthreads();
    kth = sh.best;
    __syncthreads();
    if (!use_p) { th = kth; return true; }
    u64 z = 0;
    for (int e = threadIdx.x; e < n; e += blockDim.x) z += lkey[e] >= kth ? lmass[e] : 0ull;
    z = block_sum_u64(z, sh.wsum);
    need = share_of(p, z);
    if (threadIdx.x == 0) sh.best = 0xffffffffu;
    __syncthreads();
  }
  // top-p: the smallest kept key with less than the wanted mass above it
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const uint32_t key = lkey[e];
    if (key < kth) continue;
    u64 m = above;
    for (int j = 0; j < n; ++j) m += lkey[j] > key ? lmass[j] : 0ull;
    if (m < need) atomicMin(&sh.best, key);
  }
  __syncthreads();
  th = sh.best;
  return true;
}

// One pass over the row per bit of the key: for rows that the lists above do not hold.
__device__ uint32_t threshold_bisected(const float* __restrict__ row, int vocab, float mx, float T, int k, float p,
                                       bool use_k, bool use_p, float* fscratch, int* iscratch) {
  const float invT = 1.f / T;
  // top-k: largest key such that count(key' >= key) >= k, by bisection on the ordered bits
  uint32_t kth = 0;
  if (use_k) {
    uint32_t lo = 0, hi = 0xffffffffu;   // invariant: count(>= lo) >= k
    while (lo < hi) {
      const uint32_t mid = lo + (uint32_t)(((uint64_t)hi - lo + 1) >> 1);
      int c = 0;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x) c += order_key(row[i]) >= mid;
      c = block_count(c, iscratch);
      if (c >= k) lo = mid; else hi = mid - 1;
    }
    kth = lo;
  }
  // top-p among the kept: smallest key such that mass(key' > key) < p * Z
  uint32_t pth = kth;
  if (use_p) {
    float z = 0.f;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x)
      if (order_key(row[i]) >= kth) z += expf((row[i] - mx) * invT);
    z = block_sum(z, fscratch);
    const float target = p * z;
    uint32_t lo = kth, hi = order_key(mx);   // mass(> hi) = 0 < target: hi always satisfies
    while (lo < hi) {
      const uint32_t mid = lo + ((hi - lo) >> 1);
      float sm = 0.f;
      for (int i = threadIdx.x; i < vocab; i += blockDim.x)
        if (order_key(row[i]) > mid) sm += expf((row[i] - mx) * invT);
      sm = block_sum(sm, fscratch);
      if (sm < target) hi = mid; else lo = mid + 1;
    }
    pth = lo;
  }
  return pth;
}

__global__ void __launch_bounds__(THREADS)
threshold_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                 const int* __restrict__ top_k, const float* __restrict__ top_p, uint32_t* __restrict__ threshold) {
  bspec::pdl_prologue(11);
  __shared__ ThresholdShared sh;
  const int r = blockIdx.x;
  const float T = temperature[r];
  const int k = top_k[r];
  const float p = top_p[r];
  const bool use_k = k > 0 && k < vocab, use_p = p > 0.f && p < 1.f;
  if (!(T > 0.f) || (!use_k && !use_p)) {
    if (threadIdx.x == 0) threshold[r] = 0u;
    return;
  }
  const float* row = logits + (size_t)r * vocab;
  float mx = -INFINITY, mn = INFINITY;   // the smallest of the finite ones: masked tokens do not stretch the bins
  for_each_logit(row, vocab, [&](float x) {
    mx = fmaxf(mx, x);
    if (x > -INFINITY) mn = fminf(mn, x);
  });
  mx = warp_max(mx);
  mn = -warp_max(-mn);
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if (lane == 0) { sh.fscratch[warp] = mx; sh.fscratch[32 + warp] = -mn; }
    __syncthreads();
    mx = warp_max(lane < nw ? sh.fscratch[lane] : -INFINITY);
    mn = -warp_max(lane < nw ? sh.fscratch[32 + lane] : -INFINITY);
    __syncthreads();
  }
  uint32_t th = 0;
  const bool binned = mx < INFINITY && mn < mx && threshold_binned(row, vocab, mx, mn, T, k, p, use_k, use_p, sh, th);
  if (!binned) th = threshold_bisected(row, vocab, mx, T, k, p, use_k, use_p, sh.fscratch, sh.iscratch);
  if (threadIdx.x == 0) threshold[r] = th;
}

// Stage 2 (grid: slices x rows): best of (logit / T + Gumbel noise) over one slice of the row's kept tokens;
// greedy rows (T <= 0) take the plain logit.  threshold / stream_id / counter may be null (argmax only).
constexpr int PICK_THREADS = 256;
__global__ void __launch_bounds__(PICK_THREADS)
pick_partial_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                    const uint32_t* __restrict__ threshold, const long long* __restrict__ stream_id,
                    const long long* __restrict__ counter, unsigned long long seed, float* __restrict__ part_v,
                    int* __restrict__ part_i) {
  bspec::pdl_prologue(12);
  __shared__ ArgBest scratch[32];
  const int r = blockIdx.y, nb = gridDim.x;
  const float* row = logits + (size_t)r * vocab;
  const float T = temperature != nullptr ? temperature[r] : 0.f;
  const bool greedy = !(T > 0.f);
  const float invT = greedy ? 1.f : 1.f / T;
  const uint32_t th = (threshold != nullptr && !greedy) ? threshold[r] : 0u;
  const unsigned long long sid = greedy ? 0ull : (unsigned long long)stream_id[r];
  const unsigned long long ctr = greedy ? 0ull : (unsigned long long)counter[r];
  const int per = (vocab + nb - 1) / nb;
  const int begin = blockIdx.x * per, end = min(vocab, begin + per);
  ArgBest b{-INFINITY, 0x7fffffff};
  for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
    const float x = row[i];
    if (greedy) {
      b = better(b, ArgBest{x, i});
    } else if (order_key(x) >= th) {
      const float u = uniform01(seed, sid, ctr, (uint32_t)i);
      b = better(b, ArgBest{x * invT - logf(-logf(u)), i});
    }
  }
  b = block_argmax(b, scratch);
  if (threadIdx.x == 0) {
    part_v[r * nb + blockIdx.x] = b.v;
    part_i[r * nb + blockIdx.x] = b.i;
  }
}

// Stage 3 (one warp per row): best of the slices.
__global__ void pick_final_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int nb,
                                  int* __restrict__ out) {
  bspec::pdl_prologue(13);
  const int r = blockIdx.x;
  ArgBest b{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < nb; i += 32) b = better(b, ArgBest{part_v[r * nb + i], part_i[r * nb + i]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgBest y{__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
    b = better(b, y);
  }
  if (threadIdx.x == 0) out[r] = b.i;
}
}  // namespace

// Number of slices a row is cut into for stage 2; scratch needs rows * slices floats and ints.
BSPEC_API int bspec_pick_slices(int vocab) {
  const int nb = (vocab + 4095) / 4096;
  return nb < 1 ? 1 : (nb > 32 ? 32 : nb);
}

BSPEC_API int bspec_argmax(const float* logits, int rows, int vocab, float* part_v, int* part_i, int* out,
                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rows > 65535) return (int)cudaErrorInvalidConfiguration;
  const int nb = bspec_pick_slices(vocab);
  BSPEC_LAUNCH((pick_partial_kernel), dim3(nb, rows), PICK_THREADS, 0, stream, logits, vocab, nullptr, nullptr, nullptr, nullptr,
                                                                    0ull, part_v, part_i);
  BSPEC_LAUNCH((pick_final_kernel), rows, 32, 0, stream, part_v, part_i, nb, out);
  return BSPEC_LAUNCH_CHECK();
}

// threshold: scratch uint32 [rows]; part_v / part_i: scratch [rows * bspec_pick_slices(vocab)].
BSPEC_API int bspec_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
                           const float* top_p, const long long* stream_id, const long long* counter,
                           unsigned long long seed, uint32_t* threshold, float* part_v, int* part_i, int* out,
                           cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (rows > 65535) return (int)cudaErrorInvalidConfiguration;
  const int nb = bspec_pick_slices(vocab);
  BSPEC_LAUNCH((threshold_kernel), rows, THREADS, 0, stream, logits, vocab, temperature, top_k, top_p, threshold);
  BSPEC_LAUNCH((pick_partial_kernel), dim3(nb, rows), PICK_THREADS, 0, stream, logits, vocab, temperature, threshold, stream_id,
                                                                    counter, seed, part_v, part_i);
  BSPEC_LAUNCH((pick_final_kernel), rows, 32, 0, stream, part_v, part_i, nb, out);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_sampling)
