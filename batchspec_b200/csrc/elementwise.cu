// Row-wise kernels of the decoder: embedding gather, residual add + RMSNorm,
// row gather for the head, SiLU(gate)*up, rotary encoding fused with the write of
// keys and values into cache pages.  All arithmetic is float32; storage is float32
// or bfloat16 as the caller says.
#include "common.cuh"
using namespace bspec;

// ---------------------------------------------------------------- embedding
// out[t, :] = scale * table[ids[t], :]   (out is the float32 residual stream)
template <typename T>
__global__ void embed_kernel(const int* __restrict__ ids, const T* __restrict__ table, float* __restrict__ out,
                             int d, int vocab, float scale) {
  bspec::pdl_prologue(1);
  const int t = blockIdx.x;
  int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  (void)bspec::in_range(id, vocab, 101);
  const T* row = table + (size_t)(ok ? id : 0) * d;
  float* o = out + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = ok ? to_f32(row[i]) * scale : 0.f;
}

BSPEC_API int bspec_embed(const int* ids, const void* table, int table_dtype, float* out, int n, int d, int vocab,
                          float scale, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = d >= 1024 ? 256 : 128;
  if (table_dtype == BSPEC_F32)
    BSPEC_LAUNCH((embed_kernel<float>), n, threads, 0, stream, ids, (const float*)table, out, d, vocab, scale);
  else
    BSPEC_LAUNCH((embed_kernel<__nv_bfloat16>), n, threads, 0, stream, ids, (const __nv_bfloat16*)table, out, d, vocab, scale);
  return BSPEC_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- add + RMSNorm
// resid[t,:] += delta[t,:] (if delta);  out[t,:] = cast(resid * rsqrt(mean(resid^2)+eps)) * w
// The product with w is taken after the cast to the output type, in that type.
// One block per row.  Each thread owns elements 4*(threadIdx.x + k*blockDim.x) .. +3 for k < VPT and keeps them in
// registers between the sum of squares and the scaling (one pass over memory); rows wider than
// 4 * VPT * blockDim.x, or whose width is not a multiple of 4, take the two-pass kernel below.
template <typename T> struct Vec4 { T v[4]; };
template <typename T> __device__ __forceinline__ void load4(const T* p, float (&f)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x), b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
  f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&f)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&f)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 v;
  v.x = *reinterpret_cast<const uint32_t*>(&a);
  v.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = v;
}

template <typename TD, typename TO, typename TW, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                       const TW* __restrict__ weight, TO* __restrict__ out, int d, float eps) {
  bspec::pdl_prologue(2);
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * d;
  float x[VPT][4];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = 4 * (threadIdx.x + k * blockDim.x);
    if (i < d) {
      load4<float>(resid + base + i, x[k]);
      if (delta != nullptr) {
        float dl[4];
        load4<TD>(delta + base + i, dl);
#pragma unroll
        for (int j = 0; j < 4; ++j) x[k][j] += dl[j];
        store4<float>(resid + base + i, x[k]);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) ss += x[k][j] * x[k][j];
    }
  }
  const float r = rsqrtf(block_sum(ss, scratch) / (float)d + eps);
#pragma unroll
  for (int k = 0; k < VPT; ++k) {
    const int i = 4 * (threadIdx.x + k * blockDim.x);
    if (i < d) {
      float w[4], y[4];
      load4<TW>(weight + i, w);
#pragma unroll
      for (int j = 0; j < 4; ++j) y[j] = to_f32(from_f32<TO>(to_f32(from_f32<TO>(x[k][j] * r)) * w[j]));
      store4<TO>(out + base + i, y);
    }
  }
}

template <typename TD, typename TO>
__global__ void add_rmsnorm_kernel(float* __restrict__ resid, const TD* __restrict__ delta,
                                   const void* __restrict__ weight, int w_dtype, TO* __restrict__ out, int d,
                                   float eps) {
  bspec::pdl_prologue(2);
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * d;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = resid[base + i];
    if (delta != nullptr) {
      v += to_f32(delta[base + i]);
      resid[base + i] = v;
    }
    ss += v * v;
  }
  const float total = block_sum(ss, scratch);
  const float r = rsqrtf(total / (float)d + eps);
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float n = resid[base + i] * r;
    const float w = load_as_f32(weight, w_dtype, i);
    out[base + i] = from_f32<TO>(to_f32(from_f32<TO>(n)) * w);
  }
}

template <typename TD, typename TO, typename TW>
static void launch_add_rmsnorm_vec(float* resid, const void* delta, const void* weight, void* out, int n, int d,
                                   float eps, cudaStream_t stream) {
  const int quads = d / 4;
  int threads = quads >= 1024 ? 1024 : ((quads + 31) / 32) * 32;
  // Many rows (a prompt): four quads per thread, so that a thread has more loads in flight and several rows share
  // an SM; few rows (decode): as many threads per row as there are quads, for the shortest row.  Only for bfloat16
  // output: in float32 a row's sum keeps one order of summation, whatever else is in the step.
  if (sizeof(TO) == 2 && n >= 512 && quads >= 128) threads = (((quads + 3) / 4 + 31) / 32) * 32;
  if (threads < 32) threads = 32;
  const int vpt = (quads + threads - 1) / threads;
#define LV(V) BSPEC_LAUNCH((add_rmsnorm_vec_kernel<TD, TO, TW, V>), n, threads, 0, stream, resid, (const TD*)delta, (const TW*)weight, (TO*)out, d, eps)
  if (vpt <= 1) LV(1); else if (vpt <= 2) LV(2); else LV(4);
#undef LV
}

BSPEC_API int bspec_add_rmsnorm(float* resid, const void* delta, int delta_dtype, const void* weight, int w_dtype,
                                void* out, int out_dtype, int n, int d, float eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  const bool same = delta_dtype == out_dtype;
  if (same && d % 4 == 0 && d <= 4 * 4 * 1024) {
    if (out_dtype == BSPEC_F32) {
      if (w_dtype == BSPEC_F32) launch_add_rmsnorm_vec<float, float, float>(resid, delta, weight, out, n, d, eps, stream);
      else launch_add_rmsnorm_vec<float, float, __nv_bfloat16>(resid, delta, weight, out, n, d, eps, stream);
    } else {
      if (w_dtype == BSPEC_F32) launch_add_rmsnorm_vec<__nv_bfloat16, __nv_bfloat16, float>(resid, delta, weight, out, n, d, eps, stream);
      else launch_add_rmsnorm_vec<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16>(resid, delta, weight, out, n, d, eps, stream);
    }
    return BSPEC_LAUNCH_CHECK();
  }
  const int threads = d >= 2048 ? 512 : (d >= 512 ? 256 : 128);
#define L(TD, TO) BSPEC_LAUNCH((add_rmsnorm_kernel<TD, TO>), n, threads, 0, stream, resid, (const TD*)delta, weight, w_dtype, (TO*)out, d, eps)
  if (delta_dtype == BSPEC_F32 && out_dtype == BSPEC_F32) L(float, float);
  else if (delta_dtype == BSPEC_BF16 && out_dtype == BSPEC_BF16) L(__nv_bfloat16, __nv_bfloat16);
  else if (delta_dtype == BSPEC_F32 && out_dtype == BSPEC_BF16) L(float, __nv_bfloat16);
  else L(__nv_bfloat16, float);
#undef L
  return BSPEC_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- row gather (+ pending add)
template <typename TD>
__global__ void gather_rows_add_kernel(const float* __restrict__ resid, const TD* __restrict__ pending,
                                       const int* __restrict__ rows, float* __restrict__ out, int d, int n_src) {
  bspec::pdl_prologue(3);
  if (!bspec::in_range(rows[blockIdx.x], n_src, 102)) return;
  const size_t src = (size_t)rows[blockIdx.x] * d, dst = (size_t)blockIdx.x * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = resid[src + i];
    if (pending != nullptr) v += to_f32(pending[src + i]);
    out[dst + i] = v;
  }
}

BSPEC_API int bspec_gather_rows_add(const float* resid, const void* pending, int pending_dtype, const int* rows,
                                    float* out, int n_out, int d, int n_src, cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (pending_dtype == BSPEC_F32)
    BSPEC_LAUNCH((gather_rows_add_kernel<float>), n_out, 256, 0, stream, resid, (const float*)pending, rows, out, d, n_src);
  else
    BSPEC_LAUNCH((gather_rows_add_kernel<__nv_bfloat16>), n_out, 256, 0, stream, resid, (const __nv_bfloat16*)pending, rows, out, d, n_src);
  return BSPEC_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- SiLU(gate) * up
// u [n, 2I] -> m [n, I].  group = 0: u = [gate | up] (two halves);  group = G > 0: u comes in blocks of 2G columns,
// G gate columns followed by their G up columns (the layout of the fused-epilogue GEMM's weights).
__device__ __forceinline__ size_t gate_col(size_t col, int inter, int group) {
  return group > 0 ? (col / group) * 2 * group + (col % group) : col;
}
__device__ __forceinline__ size_t up_col(size_t col, int inter, int group) {
  return group > 0 ? (col / group) * 2 * group + group + (col % group) : inter + col;
}
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ u, T* __restrict__ m, int inter, size_t total, int group) {
  bspec::pdl_prologue(4);
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (size_t)gridDim.x * blockDim.x) {
    const size_t row = idx / inter, col = idx - row * inter;
    const float g = to_f32(u[row * 2 * inter + gate_col(col, inter, group)]);
    const float up = to_f32(u[row * 2 * inter + up_col(col, inter, group)]);
    const float s = g / (1.f + expf(-g));
    m[idx] = from_f32<T>(s * up);
  }
}

// the same, eight bfloat16 per thread (I, and the group if any, multiples of 8): grid.x over the columns, grid.y
// over the rows (no 64-bit divisions per element), the exponential and the quotient in their fast forms (their
// error is far below bfloat16's step)
__global__ void silu_mul_bf16x8_kernel(const __nv_bfloat16* __restrict__ u, __nv_bfloat16* __restrict__ m, int inter,
                                       int n, int group) {
  bspec::pdl_prologue(4);
  const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
  if (c8 * 8 >= inter) return;
  const int col = c8 * 8;
  const int gcol = group > 0 ? (col / group) * 2 * group + (col % group) : col;
  const int ucol = group > 0 ? gcol + group : inter + col;
  for (int row = blockIdx.y; row < n; row += gridDim.y) {
    const __nv_bfloat16* src = u + (size_t)row * 2 * inter;
    const uint4 gv = *reinterpret_cast<const uint4*>(src + gcol);
    const uint4 uv = *reinterpret_cast<const uint4*>(src + ucol);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
    uint4 ov;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float ga = __low2float(g2[j]), gb = __high2float(g2[j]);
      const float sa = __fdividef(ga, 1.f + __expf(-ga)), sb = __fdividef(gb, 1.f + __expf(-gb));
      o2[j] = __floats2bfloat162_rn(sa * __low2float(u2[j]), sb * __high2float(u2[j]));
    }
    *reinterpret_cast<uint4*>(m + (size_t)row * inter + col) = ov;
  }
}

BSPEC_API int bspec_silu_mul(const void* u, void* m, int dtype, int n, int inter, int group, cudaStream_t stream) {
  const size_t total = (size_t)n * inter;
  if (total == 0) return 0;
  const int threads = 256;
  if (group < 0 || (group > 0 && inter % group != 0)) return (int)cudaErrorInvalidValue;
  if (dtype == BSPEC_BF16 && inter % 8 == 0 && group % 8 == 0) {
    const int inter8 = inter / 8;
    const int tx = inter8 >= 256 ? 256 : ((inter8 + 31) / 32) * 32;
    const dim3 grid((inter8 + tx - 1) / tx, n > 32768 ? 32768 : n);
    BSPEC_LAUNCH((silu_mul_bf16x8_kernel), grid, tx, 0, stream, (const __nv_bfloat16*)u, (__nv_bfloat16*)m, inter, n,
                 group);
    return BSPEC_LAUNCH_CHECK();
  }
  size_t want = (total + threads - 1) / threads;
  const size_t cap = (size_t)bspec::sm_count() * 32;
  const int blocks = (int)(want > cap ? cap : want);
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((silu_mul_kernel<float>), blocks, threads, 0, stream, (const float*)u, (float*)m, inter, total, group);
  else
    BSPEC_LAUNCH((silu_mul_kernel<__nv_bfloat16>), blocks, threads, 0, stream, (const __nv_bfloat16*)u,
                 (__nv_bfloat16*)m, inter, total, group);
  return BSPEC_LAUNCH_CHECK();
}

// ---------------------------------------------------------------- rotary + cache append
// qkv [n, (Hq + 2 Hkv) * hd]: rotate the q heads in place; rotate the k heads and
// write them, with the v heads, into the cache page of each token's position.
// Cache layer layout: [pages][2 (k, v)][Hkv][page_size][hd].
// Pairing: half-split (j, j + rot/2) or interleaved (2j, 2j+1); dims >= rot pass through.
constexpr int ROPE_HEADS_PER_BLOCK = 4;

// Sine and cosine of position * frequency j.  The table holds every frequency as two floats, [rot/2] leading
// parts then [rot/2] remainders, whose sum is the float64 frequency to 2^-48: the product and its reduction to
// [-pi, pi] are float64, so the angle is right to ~2e-7 rad (the rounding of the reduced angle to float32) at
// any position, where a float32 product would be off by position * 6e-8 rad (8e-3 rad at position 131,071).
// Sine, cosine and the rotation are float32.  A block computes rot/2 of these per token, so the cost is nil.
__device__ __forceinline__ void rope_sincos(int pos, const float* __restrict__ inv_freq, int half, int j, float* s,
                                            float* c) {
  const double f = (double)inv_freq[j] + (double)inv_freq[half + j];
  double a = (double)pos * f;
  a -= 6.283185307179586476925286766559 * rint(a * 0.15915494309189533576888376337251);
  sincosf((float)a, s, c);
}

template <typename T>
__global__ void rope_kv_append_kernel(T* __restrict__ qkv, int Hq, int Hkv, int hd, const float* __restrict__ inv_freq,
                                      int rot, int interleaved, const int* __restrict__ positions,
                                      const int* __restrict__ tok_entry, const int* __restrict__ kv_indptr,
                                      const int* __restrict__ kv_indices, T* __restrict__ cache, int page_size,
                                      int write_kv, long long n_pages) {
  bspec::pdl_prologue(5);
  extern __shared__ float cs[];  // [rot/2] cos, [rot/2] sin
  const int t = blockIdx.x;
  const int slot0 = blockIdx.y * ROPE_HEADS_PER_BLOCK;          // head slots: q heads, then k heads, then v heads
  const int n_slots = Hq + 2 * Hkv;
  const int slot1 = min(n_slots, slot0 + ROPE_HEADS_PER_BLOCK);
  const int pos = positions[t];
  const int half = rot / 2;
  if (slot0 < Hq + Hkv) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float s, c;
      rope_sincos(pos, inv_freq, half, j, &s, &c);
      cs[j] = c;
      cs[half + j] = s;
    }
  }
  __syncthreads();
  T* row = qkv + (size_t)t * n_slots * hd;
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (write_kv && slot1 > Hq) {
    const int e = tok_entry[t];
    if (bspec::in_range(pos / page_size, kv_indptr[e + 1] - kv_indptr[e], 103)) {
      const int page = kv_indices[kv_indptr[e] + pos / page_size];
      if (bspec::in_range(page, n_pages, 104)) {
        const int r = pos % page_size;
        const size_t page_elems = (size_t)Hkv * page_size * hd;
        kdst = cache + ((size_t)page * 2) * page_elems + (size_t)r * hd;
        vdst = kdst + page_elems;
      }
    }
  }
  write_kv = kdst != nullptr;
  const int hp = hd / 2;  // work items per head: one per pair of dims
  for (int w = threadIdx.x; w < (slot1 - slot0) * hp; w += blockDim.x) {
    const int h = slot0 + w / hp, j = w % hp;
    T* x = row + (size_t)h * hd;
    if (h >= Hq + Hkv) {                       // a v head: copy two elements
      if (write_kv) {
        T* vd = vdst + (size_t)(h - Hq - Hkv) * page_size * hd;
        vd[2 * j] = x[2 * j];
        vd[2 * j + 1] = x[2 * j + 1];
      }
      continue;
    }
    int a, b;
    bool rotate;
    if (j < half) {
      rotate = true;
      a = interleaved ? 2 * j : j;
      b = interleaved ? 2 * j + 1 : j + half;
    } else {  // pass-through dims rot .. hd-1, two at a time
      rotate = false;
      a = rot + 2 * (j - half);
      b = a + 1;
    }
    float xa = to_f32(x[a]), xb = to_f32(x[b]);
    if (rotate) {
      const float c = cs[j], sn = cs[half + j];
      const float ra = xa * c - xb * sn, rb = xa * sn + xb * c;
      xa = ra;
      xb = rb;
    }
    const T ya = from_f32<T>(xa), yb = from_f32<T>(xb);
    if (h < Hq) {
      if (rotate) { x[a] = ya; x[b] = yb; }
    } else if (write_kv) {
      T* kd = kdst + (size_t)(h - Hq) * page_size * hd;
      kd[a] = ya;
      kd[b] = yb;
    }
  }
}

// The same for bfloat16 rows with the half-split pairing over the whole head (rot == hd, hd a multiple of 16): every
// thread rotates eight neighbouring dims of the first half with their partners in the second half through 16-byte
// loads and stores; v heads are copied 16 bytes at a time.  One block per (token, share of the token's work).
__global__ void __launch_bounds__(256)
rope_kv_append_vec_kernel(__nv_bfloat16* __restrict__ qkv, int Hq, int Hkv, int hd, const float* __restrict__ inv_freq,
                          const int* __restrict__ positions, const int* __restrict__ tok_entry,
                          const int* __restrict__ kv_indptr, const int* __restrict__ kv_indices,
                          __nv_bfloat16* __restrict__ cache, int page_size, int write_kv, long long n_pages) {
  bspec::pdl_prologue(5);
  extern __shared__ float cs[];  // [hd/2] cos, [hd/2] sin
  const int t = blockIdx.x, half = hd / 2;
  const int pos = positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    rope_sincos(pos, inv_freq, half, j, &s, &c);
    cs[j] = c;
    cs[half + j] = s;
  }
  __syncthreads();
  const int n_slots = Hq + 2 * Hkv;
  __nv_bfloat16* row = qkv + (size_t)t * n_slots * hd;
  __nv_bfloat16* kdst = nullptr;
  __nv_bfloat16* vdst = nullptr;
  if (write_kv) {
    const int e = tok_entry[t];
    if (bspec::in_range(pos / page_size, kv_indptr[e + 1] - kv_indptr[e], 103)) {
      const int page = kv_indices[kv_indptr[e] + pos / page_size];
      if (bspec::in_range(page, n_pages, 104)) {
        const size_t page_elems = (size_t)Hkv * page_size * hd;
        kdst = cache + ((size_t)page * 2) * page_elems + (size_t)(pos % page_size) * hd;
        vdst = kdst + page_elems;
      }
    }
    write_kv = kdst != nullptr;
  }
  const int per_rot = half / 8;                 // items per rotated head: eight pairs each
  const int n_rot = (Hq + Hkv) * per_rot;
  const int per_v = hd / 8;                     // items per v head: eight elements each
  const int n_items = n_rot + (write_kv ? Hkv * per_v : 0);
  for (int w = blockIdx.y * blockDim.x + threadIdx.x; w < n_items; w += gridDim.y * blockDim.x) {
    if (w >= n_rot) {
      const int h = (w - n_rot) / per_v, c8 = (w - n_rot) - h * per_v;
      *reinterpret_cast<uint4*>(vdst + (size_t)h * page_size * hd + 8 * c8) =
          *reinterpret_cast<const uint4*>(row + (size_t)(Hq + Hkv + h) * hd + 8 * c8);
      continue;
    }
    const int h = w / per_rot, j0 = 8 * (w - h * per_rot);
    __nv_bfloat16* x = row + (size_t)h * hd;
    const uint4 lo = *reinterpret_cast<const uint4*>(x + j0), hi = *reinterpret_cast<const uint4*>(x + half + j0);
    const __nv_bfloat16* a = reinterpret_cast<const __nv_bfloat16*>(&lo);
    const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(&hi);
    uint4 out_lo, out_hi;
    __nv_bfloat16* ya = reinterpret_cast<__nv_bfloat16*>(&out_lo);
    __nv_bfloat16* yb = reinterpret_cast<__nv_bfloat16*>(&out_hi);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float xa = __bfloat162float(a[i]), xb = __bfloat162float(b[i]);
      const float c = cs[j0 + i], sn = cs[half + j0 + i];
      ya[i] = __float2bfloat16_rn(xa * c - xb * sn);
      yb[i] = __float2bfloat16_rn(xa * sn + xb * c);
    }
    if (h < Hq) {
      *reinterpret_cast<uint4*>(x + j0) = out_lo;
      *reinterpret_cast<uint4*>(x + half + j0) = out_hi;
    } else if (write_kv) {
      __nv_bfloat16* kd = kdst + (size_t)(h - Hq) * page_size * hd;
      *reinterpret_cast<uint4*>(kd + j0) = out_lo;
      *reinterpret_cast<uint4*>(kd + half + j0) = out_hi;
    }
  }
}

BSPEC_API int bspec_rope_kv_append(void* qkv, int dtype, int n, int Hq, int Hkv, int hd, const float* inv_freq, int rot,
                                   int interleaved, const int* positions, const int* tok_entry, const int* kv_indptr,
                                   const int* kv_indices, void* cache, int page_size, int write_kv,
                                   long long n_pages, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = 128;
  const size_t smem = (size_t)(rot > 0 ? rot : 0) * sizeof(float);
  if (dtype == BSPEC_BF16 && rot == hd && !interleaved && hd % 16 == 0 && n >= 64 &&
      (reinterpret_cast<uintptr_t>(qkv) & 15) == 0 && (reinterpret_cast<uintptr_t>(cache) & 15) == 0) {
    // many tokens: one block per token (or two while they are few) with 16-byte accesses
    BSPEC_LAUNCH((rope_kv_append_vec_kernel), dim3(n, n >= 512 ? 1 : 2), 256, smem, stream, (__nv_bfloat16*)qkv, Hq, Hkv, hd,
                 inv_freq, positions, tok_entry, kv_indptr, kv_indices, (__nv_bfloat16*)cache, page_size, write_kv, n_pages);
    return BSPEC_LAUNCH_CHECK();
  }
  dim3 grid(n, (Hq + 2 * Hkv + ROPE_HEADS_PER_BLOCK - 1) / ROPE_HEADS_PER_BLOCK);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((rope_kv_append_kernel<float>), grid, threads, smem, stream, (float*)qkv, Hq, Hkv, hd, inv_freq, rot, interleaved,
                                                                 positions, tok_entry, kv_indptr, kv_indices,
                                                                 (float*)cache, page_size, write_kv, n_pages);
  else
    BSPEC_LAUNCH((rope_kv_append_kernel<__nv_bfloat16>), grid, threads, smem, stream, 
        (__nv_bfloat16*)qkv, Hq, Hkv, hd, inv_freq, rot, interleaved, positions, tok_entry, kv_indptr, kv_indices,
        (__nv_bfloat16*)cache, page_size, write_kv, n_pages);
  return BSPEC_LAUNCH_CHECK();
}

// Rotary encoding alone, on a strided view x [n, H, hd] (row stride given in elements).
template <typename T>
__global__ void rope_inplace_kernel(T* __restrict__ x, long long row_stride, int H, int hd,
                                    const float* __restrict__ inv_freq, int rot, int interleaved,
                                    const int* __restrict__ positions) {
  bspec::pdl_prologue(6);
  extern __shared__ float cs[];
  const int t = blockIdx.x, half = rot / 2;
  const int pos = positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    rope_sincos(pos, inv_freq, half, j, &s, &c);
    cs[j] = c;
    cs[half + j] = s;
  }
  __syncthreads();
  T* row = x + (size_t)t * row_stride;
  for (int w = threadIdx.x; w < H * half; w += blockDim.x) {
    const int h = w / half, j = w - h * half;
    T* p = row + (size_t)h * hd;
    const int a = interleaved ? 2 * j : j, b = interleaved ? 2 * j + 1 : j + half;
    const float xa = to_f32(p[a]), xb = to_f32(p[b]);
    const float c = cs[j], s = cs[half + j];
    p[a] = from_f32<T>(xa * c - xb * s);
    p[b] = from_f32<T>(xa * s + xb * c);
  }
}

BSPEC_API int bspec_rope_inplace(void* x, int dtype, int n, long long row_stride, int H, int hd, const float* inv_freq,
                                 int rot, int interleaved, const int* positions, cudaStream_t stream) {
  if (n <= 0 || rot <= 0) return 0;
  const size_t smem = (size_t)rot * sizeof(float);
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((rope_inplace_kernel<float>), n, 128, smem, stream, (float*)x, row_stride, H, hd, inv_freq, rot, interleaved, positions);
  else
    BSPEC_LAUNCH((rope_inplace_kernel<__nv_bfloat16>), n, 128, smem, stream, (__nv_bfloat16*)x, row_stride, H, hd, inv_freq, rot, interleaved, positions);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_elementwise)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_elementwise)
