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
__global__ void __launch_bounds__(THREADS)
threshold_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                 const int* __restrict__ top_k, const float* __restrict__ top_p, uint32_t* __restrict__ threshold) {
  bspec::pdl_prologue(11);
  __shared__ float fscratch[32];
  __shared__ int iscratch[32];
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
  const float invT = 1.f / T;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, row[i]);
  mx = warp_max(mx);
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) fscratch[warp] = mx;
    __syncthreads();
    float t = lane < nw ? fscratch[lane] : -INFINITY;
    mx = warp_max(t);
  }
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
  if (threadIdx.x == 0) threshold[r] = pth;
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
