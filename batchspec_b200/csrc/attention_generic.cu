// Paged causal attention, generic path: any head_dim that is a multiple of 16 up
// to 256, any number of heads and groups, any page size, float32 or bfloat16
// storage, float32 arithmetic throughout.  One warp per (query token, query
// head); a block holds WARPS consecutive query tokens of one request and one
// head.  Keys are visited in chunks of 32 that start at multiples of 32 of the
// key index, so the order of every sum depends only on the query's own position,
// not on how the request was cut into steps or on what else is in the batch.
//
// Cache layer layout: [pages][2 (k, v)][Hkv][page_size][hd].
#include "common.cuh"
#include <math.h>
using namespace bspec;

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_generic_kernel(const T* __restrict__ q, long long q_row_stride, T* __restrict__ out,
                    const T* __restrict__ cache, const int* __restrict__ qo_indptr,
                    const int* __restrict__ positions, const int* __restrict__ kv_indptr,
                    const int* __restrict__ kv_indices, int Hq, int Hkv, int hd, int page_size, float scale,
                    int window, long long n_pages) {
  bspec::pdl_prologue(7);
  __shared__ float qs[WARPS][MAX_HD];
  const int e = blockIdx.y, h = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_begin = qo_indptr[e], q_len = qo_indptr[e + 1] - q_begin;
  const int qi = blockIdx.x * WARPS + warp;
  if (blockIdx.x * WARPS >= q_len) return;   // whole block beyond this request's tokens
  const bool active = qi < q_len;
  const int t = q_begin + (active ? qi : 0);
  const int kvh = h / (Hq / Hkv);
  if (active) {
    const T* qp = q + (size_t)t * q_row_stride + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qs[warp][d] = to_f32(qp[d]);
  }
  __syncwarp();
  if (!active) return;
  const int pos = positions[t];
  const int hi = pos;                                   // last visible key (inclusive)
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int* table = kv_indices + kv_indptr[e];
  const size_t page_elems = (size_t)Hkv * page_size * hd;
  const size_t head_off = (size_t)kvh * page_size * hd;
  constexpr int ND = MAX_HD / 32;
  float acc[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int kb = (lo / 32) * 32; kb <= hi; kb += 32) {
    const int key = kb + lane;
    bool valid = key >= lo && key <= hi;
    long long koff = 0;
    float s = -INFINITY;
    if (valid && !bspec::in_range(table[key / page_size], n_pages, 107)) valid = false;
    if (valid) {
      const int page = table[key / page_size];
      koff = (long long)((size_t)page * 2 * page_elems + head_off + (size_t)(key % page_size) * hd);
      const T* kp = cache + koff;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot += qs[warp][d] * to_f32(kp[d]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));        // finite: the chunk holds at least one valid key
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);               // m = -inf on the first chunk -> 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= corr;
    const int nk = min(32, hi - kb + 1);
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const long long off = __shfl_sync(0xffffffffu, koff, kk);
      if (pk != 0.f) {
        const T* vp = cache + off + page_elems;
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          const int d = lane + 32 * i;
          if (d < hd) acc[i] += pk * to_f32(vp[d]);
        }
      }
    }
    m = m_new;
  }
  const float inv = 1.f / l;
  T* op = out + ((size_t)t * Hq + h) * hd;
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) op[d] = from_f32<T>(acc[i] * inv);
  }
}
}  // namespace

// q: rows of row stride q_row_stride (elements), heads packed [Hq][hd] at the row start.
// out: [n, Hq*hd].  max_q_len: the longest request portion in the step (sizes the grid).
BSPEC_API int bspec_attention_generic(const void* q, long long q_row_stride, void* out, const void* cache, int dtype,
                                      const int* qo_indptr, const int* positions, const int* kv_indptr,
                                      const int* kv_indices, int n_entries, int max_q_len, int Hq, int Hkv, int hd,
                                      int page_size, float scale, int window, long long n_pages,
                                      cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return 0;
  if (hd > MAX_HD || hd <= 0 || Hq % Hkv != 0) return (int)cudaErrorInvalidValue;
  dim3 grid((max_q_len + WARPS - 1) / WARPS, n_entries, Hq);
  if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidConfiguration;
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((attn_generic_kernel<float>), grid, WARPS * 32, 0, stream, 
        (const float*)q, q_row_stride, (float*)out, (const float*)cache, qo_indptr, positions, kv_indptr, kv_indices,
        Hq, Hkv, hd, page_size, scale, window, n_pages);
  else
    BSPEC_LAUNCH((attn_generic_kernel<__nv_bfloat16>), grid, WARPS * 32, 0, stream, 
        (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)cache, qo_indptr, positions,
        kv_indptr, kv_indices, Hq, Hkv, hd, page_size, scale, window, n_pages);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_attention_generic)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_attention_generic)
