// Kernels of layers that cache a low-rank latent instead of per-head keys and values, and of the
// arrangements such models use around their sublayers.  All arithmetic is float32; the element
// type of activations and of the cache (float or bfloat16) is a template parameter.
//
//  * scale_cast:        y = alpha * x (float32), h = T(x): the two readers of a stream whose norm
//                       comes after the sum (the sublayer reads h, its output is added to y).
//  * sum_norm:          x = rmsnorm(y) * gain, and for the next sublayer y = alpha * x, h = T(x).
//  * polynorm:          a N(z) + b N(z^2) + c N(z^3) + e with N = division by the row's root mean square.
//  * latent_kv_append:  per token a row [latent (rank) | shared rotary key part]: the latent is
//                       RMS-normed with a learned weight, the key part rotated by the token's
//                       position, and both are stored as one row of a paged cache with one head.
//  * latent_query_tail: the rotated part of every query head, copied behind the head's latent
//                       query (the row a latent attention kernel multiplies with a cache row).
//  * headwise_gemm:     out[t, h, :] = W[h] a[t, h, :], one small matrix per head.
//  * latent_attention_simple: causal attention of (token, head) rows over the latent cache rows,
//                       all heads reading the same row; the value is the row's first `rank`
//                       elements; optional sink term in the softmax denominator.
//  * depth_average:     keeps a layer's result in a history and replaces the stream by a weighted
//                       sum of the history so far.
//  * softcap:           x = cap * tanh(x / cap), in place.
#include "attention_bf16.cuh"

using namespace sprout_attn;

namespace {

// ---------------------------------------------------------------- scale_cast
template <typename TO>
__global__ void scale_cast_kernel(const float* __restrict__ x, float* __restrict__ y, TO* __restrict__ h,
                                  float alpha, long long count) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x) {
    const float v = x[i];
    y[i] = alpha * v;
    if (h) h[i] = from_float<TO>(v);
  }
}

// ---------------------------------------------------------------- sum_norm
// One block per row.  `x` may be `y` itself; y2 may be y too (every element is read by the thread
// that later writes it).
template <typename TO>
__global__ void __launch_bounds__(256)
sum_norm_kernel(const float* y, const float* __restrict__ gain, float* x, float* y2, TO* __restrict__ h,
                int hidden, float eps, float alpha) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) { const float v = y[row + i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float v = (y[row + i] * scale) * gain[i];
    x[row + i] = v;
    if (y2) y2[row + i] = alpha * v;
    if (h) h[row + i] = from_float<TO>(v);
  }
}

// ---------------------------------------------------------------- polynorm
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
polynorm_kernel(const TI* __restrict__ z, TO* __restrict__ out, const float* __restrict__ coef, int width, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * width;
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_float(z[row + i]);
    const float v2 = v * v, v3 = v2 * v;
    s2 = fmaf(v, v, s2);
    s4 = fmaf(v2, v2, s4);
    s6 = fmaf(v3, v3, s6);
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float r1 = 1.0f / sqrtf(s2 / (float)width + eps);
  const float r2 = 1.0f / sqrtf(s4 / (float)width + eps);
  const float r3 = 1.0f / sqrtf(s6 / (float)width + eps);
  const float a = coef[0], b = coef[1], c = coef[2], e = coef[3];
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    const float v = to_float(z[row + i]);
    const float v2 = v * v, v3 = v2 * v;
    out[row + i] = from_float<TO>(a * (v * r1) + b * (v2 * r2) + c * (v3 * r3) + e);
  }
}

// Rows whose width is a multiple of 4 and at most 256 x 4 x VEC: the row stays in registers between the sums and
// the output (one read), 16-byte accesses.
template <typename TO>
__device__ __forceinline__ void store4(TO* dst, int i, float a, float b, float c, float d) {
  if (sizeof(TO) == 4) {
    ((float4*)dst)[i] = make_float4(a, b, c, d);
  } else {
    __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
    ((uint2*)dst)[i] = make_uint2(*(uint32_t*)&lo, *(uint32_t*)&hi);
  }
}

// With `history` ([entries, rows, hidden] float32): the normed row is kept as entry n + 1 and what goes on (x, y2, h) is
// sum_{j <= n + 1} w[j] * history[j] of the row, in the order the separate depth_average kernel adds.
template <typename TO, int VEC>
__global__ void __launch_bounds__(256)
sum_norm_vec_kernel(const float* y, const float* __restrict__ gain, float* x, float* y2, TO* __restrict__ h,
                    int hidden, float eps, float alpha, float* history, const float* __restrict__ w, int n, long long plane) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * hidden;
  const int quads = hidden >> 2;
  float4 v[VEC];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < VEC; k++) {
    const int i = threadIdx.x + k * 256;
    v[k] = i < quads ? ((const float4*)(y + row))[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
  }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int k = 0; k < VEC; k++) {
    const int i = threadIdx.x + k * 256;
    if (i < quads) {
      const float4 g = ((const float4*)gain)[i];
      float a = (v[k].x * scale) * g.x, b = (v[k].y * scale) * g.y, c = (v[k].z * scale) * g.z, d = (v[k].w * scale) * g.w;
      if (history) {
        ((float4*)(history + (long long)(n + 1) * plane + row))[i] = make_float4(a, b, c, d);
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int j = 0; j <= n; j++) {
          const float4 e = ((const float4*)(history + (long long)j * plane + row))[i];
          const float wj = w[j];
          sum.x = fmaf(wj, e.x, sum.x); sum.y = fmaf(wj, e.y, sum.y); sum.z = fmaf(wj, e.z, sum.z); sum.w = fmaf(wj, e.w, sum.w);
        }
        const float wl = w[n + 1];
        a = fmaf(wl, a, sum.x); b = fmaf(wl, b, sum.y); c = fmaf(wl, c, sum.z); d = fmaf(wl, d, sum.w);
      }
      ((float4*)(x + row))[i] = make_float4(a, b, c, d);
      if (y2) ((float4*)(y2 + row))[i] = make_float4(alpha * a, alpha * b, alpha * c, alpha * d);
      if (h) store4<TO>(h + row, i, a, b, c, d);
    }
  }
}

template <typename TO, int VEC>
__global__ void __launch_bounds__(256)
polynorm_vec_kernel(const float* __restrict__ z, TO* __restrict__ out, const float* __restrict__ coef, int width, float eps) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * width;
  const int quads = width >> 2;
  float4 v[VEC];
  float s2 = 0.f, s4 = 0.f, s6 = 0.f;
#pragma unroll
  for (int k = 0; k < VEC; k++) {
    const int i = threadIdx.x + k * 256;
    v[k] = i < quads ? ((const float4*)(z + row))[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    const float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const float p2 = e[j] * e[j], p3 = p2 * e[j];
      s2 = fmaf(e[j], e[j], s2);
      s4 = fmaf(p2, p2, s4);
      s6 = fmaf(p3, p3, s6);
    }
  }
  s2 = block_sum(s2, scratch);
  s4 = block_sum(s4, scratch);
  s6 = block_sum(s6, scratch);
  const float r1 = 1.0f / sqrtf(s2 / (float)width + eps);
  const float r2 = 1.0f / sqrtf(s4 / (float)width + eps);
  const float r3 = 1.0f / sqrtf(s6 / (float)width + eps);
  const float a = coef[0], b = coef[1], c = coef[2], e0 = coef[3];
#pragma unroll
  for (int k = 0; k < VEC; k++) {
    const int i = threadIdx.x + k * 256;
    if (i < quads) {
      const float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
      float r[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        const float p2 = e[j] * e[j], p3 = p2 * e[j];
        r[j] = a * (e[j] * r1) + b * (p2 * r2) + c * (p3 * r3) + e0;
      }
      store4<TO>(out + row, i, r[0], r[1], r[2], r[3]);
    }
  }
}

// ---------------------------------------------------------------- latent_kv_append
// src row t (float32, row stride ld): [rank latent values | rot shared key values].  The cache
// row of token t: page = table[seq][pos / page_tokens], slot pos % page_tokens, `rank + rot` wide.
template <typename TC>
__global__ void __launch_bounds__(128)
latent_kv_append_kernel(const float* __restrict__ src, int ld, const float* __restrict__ weight,
                        const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                        const int* __restrict__ block_table, int table_stride,
                        const float* __restrict__ cos_table, const float* __restrict__ sin_table, int table_positions,
                        int rotary_dim, int interleaved, TC* __restrict__ cache, int rank, int rot, int page_tokens,
                        int num_pages, float eps, int* status) {
  __shared__ float scratch[33];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* row = src + (size_t)t * ld;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) { const float v = row[i]; ss = fmaf(v, v, ss); }
  ss = block_sum(ss, scratch);
  const float scale = 1.0f / sqrtf(ss / (float)rank + eps);
  const int pos = positions[t];
  const int page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_tokens];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  TC* dst = cache + ((size_t)page * page_tokens + pos % page_tokens) * (rank + rot);
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_float<TC>((row[i] * scale) * weight[i]);
  const float* key = row + rank;
  const int half = rotary_dim / 2;
  int p = pos;
  if (half > 0 && (p < 0 || p >= table_positions)) {
    if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_POSITION);
    p = 0;
  }
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
    const float c = cos_table[(size_t)p * half + i], s = sin_table[(size_t)p * half + i];
    const float u = key[a], v = key[b];
    dst[rank + a] = from_float<TC>(u * c - v * s);
    dst[rank + b] = from_float<TC>(v * c + u * s);
  }
  for (int i = rotary_dim + threadIdx.x; i < rot; i += blockDim.x) dst[rank + i] = from_float<TC>(key[i]);
}

// ---------------------------------------------------------------- latent_query_tail
// q [tokens, heads, dim + rot] -> qlat[t, h, rank + (0..rot)] = rotation of q[t, h, dim + (0..rot)].
template <typename T>
__global__ void latent_query_tail_kernel(const T* __restrict__ q, T* __restrict__ qlat, const int* __restrict__ positions,
                                         const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                         int table_positions, int rotary_dim, int interleaved, int heads, int dim,
                                         int rot, int rank, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int half = rotary_dim / 2;
  int p = positions[t];
  if (half > 0 && (p < 0 || p >= table_positions)) {
    if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_POSITION);
    p = 0;
  }
  const int pairs_and_rest = half + (rot - rotary_dim);
  for (int idx = threadIdx.x; idx < heads * pairs_and_rest; idx += blockDim.x) {
    const int h = idx / pairs_and_rest, i = idx % pairs_and_rest;
    const T* src = q + ((size_t)t * heads + h) * (dim + rot) + dim;
    T* dst = qlat + ((size_t)t * heads + h) * (rank + rot) + rank;
    if (i < half) {
      const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
      const float c = cos_table[(size_t)p * half + i], s = sin_table[(size_t)p * half + i];
      const float u = to_float(src[a]), v = to_float(src[b]);
      dst[a] = from_float<T>(u * c - v * s);
      dst[b] = from_float<T>(v * c + u * s);
    } else {
      const int d = rotary_dim + (i - half);
      dst[d] = src[d];
    }
  }
}

// ---------------------------------------------------------------- headwise_gemm
// out[t, h, n] = sum_k a[t, h, k] * w[h, n, k]; one thread per output element group, ascending k,
// so a value does not depend on the number of rows in the call.
constexpr int HB = 64, HK = 16, HTHREADS = 256;

template <typename T>
__global__ void __launch_bounds__(HTHREADS)
headwise_gemm_kernel(const T* __restrict__ A, long long a_row, long long a_head, const T* __restrict__ W,
                     T* __restrict__ out, long long o_row, long long o_head, int M, int N, int K) {
  __shared__ float As[HK][HB + 4];
  __shared__ float Ws[HK][HB + 4];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, ty = tid / 16, tx = tid % 16;
  const int head = blockIdx.z;
  const int m0 = blockIdx.y * HB, n0 = blockIdx.x * HB;
  const T* a = A + head * a_head;
  const T* w = W + (size_t)head * N * K;
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; i++)
#pragma unroll
    for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += HK) {
#pragma unroll
    for (int i = 0; i < (HB * HK) / HTHREADS; i++) {
      const int idx = tid + i * HTHREADS;
      const int row = idx / HK, k = idx % HK;
      const int gm = m0 + row, gn = n0 + row, gk = k0 + k;
      As[k][row] = (gm < M && gk < K) ? to_float(a[(size_t)gm * a_row + gk]) : 0.f;
      Ws[k][row] = (gn < N && gk < K) ? to_float(w[(size_t)gn * K + gk]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < HK; k++) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; i++) av[i] = As[k][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; j++) wv[j] = Ws[k][tx * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int gm = m0 + ty * 4 + i;
    if (gm >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; j++) {
      const int gn = n0 + tx * 4 + j;
      if (gn < N) out[(size_t)gm * o_row + head * o_head + gn] = from_float<T>(acc[i][j]);
    }
  }
}

// The same on tensor cores (bfloat16): a CTA makes 64 rows x 64 columns of one head, 4 warps of 16 rows each,
// K in steps of 32 through shared memory (ldmatrix, mma.sync.m16n8k16, float32 accumulation).
constexpr int TB = 64, TK = 32, TSTRIDE = TK + 8;

__global__ void __launch_bounds__(128)
headwise_gemm_mma_kernel(const __nv_bfloat16* __restrict__ A, long long a_row, long long a_head,
                         const __nv_bfloat16* __restrict__ W, __nv_bfloat16* __restrict__ out, long long o_row,
                         long long o_head, int M, int N, int K) {
  __shared__ __align__(16) __nv_bfloat16 As[2][TB][TSTRIDE];
  __shared__ __align__(16) __nv_bfloat16 Ws[2][TB][TSTRIDE];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int head = blockIdx.z, m0 = blockIdx.y * TB, n0 = blockIdx.x * TB;
  const __nv_bfloat16* a = A + head * a_head;
  const __nv_bfloat16* w = W + (size_t)head * N * K;
  float acc[8][4];
#pragma unroll
  for (int i = 0; i < 8; i++) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
  auto load = [&](int buf, int k0) {
#pragma unroll
    for (int i = 0; i < 2; i++) {
      const int idx = tid + i * 128, row = idx >> 2, c = (idx & 3) * 8;
      const bool in_k = k0 + c < K;
      if (m0 + row < M && in_k) cp_async16(&As[buf][row][c], a + (size_t)(m0 + row) * a_row + k0 + c);
      else *(uint4*)&As[buf][row][c] = make_uint4(0, 0, 0, 0);
      if (n0 + row < N && in_k) cp_async16(&Ws[buf][row][c], w + (size_t)(n0 + row) * K + k0 + c);
      else *(uint4*)&Ws[buf][row][c] = make_uint4(0, 0, 0, 0);
    }
  };
  const int steps = (K + TK - 1) / TK;
  load(0, 0);
  cp_async_commit();
  for (int t = 0; t < steps; t++) {
    const int buf = t & 1;
    if (t + 1 < steps) load(buf ^ 1, (t + 1) * TK);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < TK / 16; kk++) {
      uint32_t af[4];
      ldmatrix_x4(af, &As[buf][warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8][kk * 16 + (lane >> 4) * 8]);
#pragma unroll
      for (int n2 = 0; n2 < 4; n2++) {
        uint32_t b[4];
        ldmatrix_x4(b, &Ws[buf][n2 * 16 + (lane & 7) + (lane >> 4) * 8][kk * 16 + ((lane >> 3) & 1) * 8]);
        mma_bf16(acc[2 * n2], af, b[0], b[1]);
        mma_bf16(acc[2 * n2 + 1], af, b[2], b[3]);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  const int gr = lane >> 2, qc = lane & 3;
#pragma unroll
  for (int half = 0; half < 2; half++) {
    const int gm = m0 + warp * 16 + gr + half * 8;
    if (gm >= M) continue;
    __nv_bfloat16* dst = out + (size_t)gm * o_row + head * o_head;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      const int gn = n0 + i * 8 + qc * 2;
      if (gn < N) *(__nv_bfloat162*)(dst + gn) = __floats2bfloat162_rn(acc[i][half * 2], acc[i][half * 2 + 1]);
    }
  }
}

// ---------------------------------------------------------------- latent_attention_simple
// One block per (token, head).  Keys are walked in chunks of 128 aligned to absolute position with a
// running maximum and sum that start from the head's sink (maximum = sink, sum = 1) when one is given.
constexpr int CHUNK = 128;
constexpr int MAX_V = 8;     // value elements per thread: rank <= MAX_V * CHUNK

template <typename T>
__global__ void __launch_bounds__(CHUNK)
latent_attention_simple_kernel(const T* __restrict__ qlat, const T* __restrict__ cache,
                               const int* __restrict__ block_table, int table_stride,
                               const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                               const float* __restrict__ sink, T* __restrict__ out, int heads, int width, int rank,
                               int page_tokens, int num_pages, float scale, int* status) {
  extern __shared__ float smem[];
  float* qs = smem;                       // width
  float* probs = qs + width;              // CHUNK
  float* scratch = probs + CHUNK;         // 34
  long long* row_offset = (long long*)(scratch + 34 + ((width & 1) ? 1 : 0));
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  for (int d = tid; d < width; d += CHUNK) qs[d] = to_float(qlat[((size_t)t * heads + h) * width + d]);
  __syncthreads();
  float m_run = sink ? sink[h] : -INFINITY, l_run = sink ? 1.f : 0.f;
  float acc[MAX_V];
#pragma unroll
  for (int i = 0; i < MAX_V; i++) acc[i] = 0.f;
  for (int base = 0; base <= pos; base += CHUNK) {
    const int p = base + tid;
    bool valid = p <= pos;
    long long offset = 0;
    if (valid) {
      const int page = table[p / page_tokens];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, SPROUT_STATUS_BAD_PAGE);
        valid = false;
      } else {
        offset = ((long long)page * page_tokens + (p % page_tokens)) * width;
      }
    }
    float s = -INFINITY;
    if (valid) {
      const T* key = cache + offset;
      float dot = 0.f;
      for (int d = 0; d < width; d++) dot = fmaf(qs[d], to_float(key[d]), dot);
      s = dot * scale;
    }
    row_offset[tid] = valid ? offset : -1;
    const float c_max = block_max(s, scratch);
    const float m_new = fmaxf(m_run, c_max);
    const float e = valid ? expf(s - m_new) : 0.f;
    probs[tid] = e;
    const float c_sum = block_sum(e, scratch);
    const float alpha = (m_run == -INFINITY) ? 0.f : expf(m_run - m_new);
    l_run = l_run * alpha + c_sum;
    const int count = min(CHUNK, pos - base + 1);
#pragma unroll
    for (int i = 0; i < MAX_V; i++) {
      const int d = tid + i * CHUNK;
      if (d < rank) {
        float a = acc[i] * alpha;
        for (int j = 0; j < count; j++) {
          const long long off = row_offset[j];
          if (off >= 0) a = fmaf(probs[j], to_float(cache[off + d]), a);
        }
        acc[i] = a;
      }
    }
    m_run = m_new;
    __syncthreads();
  }
  T* dst = out + ((size_t)t * heads + h) * rank;
#pragma unroll
  for (int i = 0; i < MAX_V; i++) {
    const int d = tid + i * CHUNK;
    if (d < rank) dst[d] = from_float<T>(acc[i] / l_run);
  }
}

// ---------------------------------------------------------------- depth_average
// history [entries, rows, width] float32.  history[n + 1] = x; x = sum_{j <= n + 1} w[j] * history[j].
__global__ void depth_average_kernel(float* __restrict__ history, float* __restrict__ x, const float* __restrict__ w,
                                     int n, long long plane) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < plane; i += (long long)gridDim.x * blockDim.x) {
    const float latest = x[i];
    history[(long long)(n + 1) * plane + i] = latest;
    float sum = 0.f;
    for (int j = 0; j <= n; j++) sum = fmaf(w[j], history[(long long)j * plane + i], sum);
    x[i] = fmaf(w[n + 1], latest, sum);
  }
}

__global__ void depth_average_vec_kernel(float4* __restrict__ history, float4* __restrict__ x, const float* __restrict__ w,
                                         int n, long long plane4) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < plane4; i += (long long)gridDim.x * blockDim.x) {
    const float4 latest = x[i];
    history[(long long)(n + 1) * plane4 + i] = latest;
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int j = 0; j <= n; j++) {
      const float4 v = history[(long long)j * plane4 + i];
      const float wj = w[j];
      sum.x = fmaf(wj, v.x, sum.x); sum.y = fmaf(wj, v.y, sum.y); sum.z = fmaf(wj, v.z, sum.z); sum.w = fmaf(wj, v.w, sum.w);
    }
    const float wl = w[n + 1];
    x[i] = make_float4(fmaf(wl, latest.x, sum.x), fmaf(wl, latest.y, sum.y), fmaf(wl, latest.z, sum.z), fmaf(wl, latest.w, sum.w));
  }
}

__global__ void softcap_kernel(float* __restrict__ x, float cap, long long count) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count; i += (long long)gridDim.x * blockDim.x)
    x[i] = cap * tanhf(x[i] / cap);
}

inline int flat_grid(long long count, int threads) {
  long long blocks = (count + threads - 1) / threads;
  const long long cap = (long long)sprout_sm_count() * 16;
  return (int)(blocks < 1 ? 1 : blocks > cap ? cap : blocks);
}

}  // namespace

SPROUT_API int sprout_scale_cast(const float* x, float* y, void* h, int h_dtype, float alpha, long long count,
                                 cudaStream_t stream) {
  SPROUT_REQUIRE(x && y && count > 0, "scale_cast: null pointer or no elements");
  if (h && h_dtype == SPROUT_BF16)
    sprout_launch(scale_cast_kernel<__nv_bfloat16>, dim3(flat_grid(count, 256)), dim3(256), 0, stream, x, y, (__nv_bfloat16*)h, alpha, count);
  else
    sprout_launch(scale_cast_kernel<float>, dim3(flat_grid(count, 256)), dim3(256), 0, stream, x, y, (float*)h, alpha, count);
  return sprout_check_launch("scale_cast");
}

SPROUT_API int sprout_scale_cast(const float* x, float* y, void* h, int h_dtype, float alpha, long long count, cudaStream_t stream);
SPROUT_API int sprout_depth_average(float* history, float* x, const float* weights, int n, long long plane, cudaStream_t stream);

// x = rmsnorm(y) * gain; optionally y2 = alpha * x and h = x in h's dtype.  With `history` (float32 [entries, rows, hidden])
// and `weights`: the normed rows become entry n + 1 of the history, and x (and y2, h) is the weighted sum of the entries
// 0..n+1: the norm after a layer's last sum, the depth average and the next layer's readers in one launch.
SPROUT_API int sprout_sum_norm(const float* y, const float* gain, float* x, float* y2, void* h, int h_dtype, int rows,
                               int hidden, float eps, float alpha, float* history, const float* weights, int n,
                               cudaStream_t stream) {
  SPROUT_REQUIRE(y && gain && x && rows > 0 && hidden > 0, "sum_norm: null pointer or empty");
  SPROUT_REQUIRE(!history || (weights && n >= 0), "sum_norm: a history comes with its weights");
  const long long plane = (long long)rows * hidden;
  const bool aligned = hidden % 4 == 0 && hidden <= 8192 &&
                       (((uintptr_t)y | (uintptr_t)gain | (uintptr_t)x | (uintptr_t)y2 | (uintptr_t)h | (uintptr_t)history) & 15) == 0;
  if (aligned) {
#define SUM_NORM_VEC(TO, VEC) sprout_launch(sum_norm_vec_kernel<TO, VEC>, dim3(rows), dim3(256), 0, stream, y, gain, x, y2, (TO*)h, hidden, eps, alpha, history, weights, n, plane)
#define SUM_NORM_PICK(TO) do { if (hidden <= 1024) SUM_NORM_VEC(TO, 1); else if (hidden <= 2048) SUM_NORM_VEC(TO, 2); \
                               else if (hidden <= 4096) SUM_NORM_VEC(TO, 4); else SUM_NORM_VEC(TO, 8); } while (0)
    if (h && h_dtype == SPROUT_BF16) SUM_NORM_PICK(__nv_bfloat16); else SUM_NORM_PICK(float);
#undef SUM_NORM_PICK
#undef SUM_NORM_VEC
    return sprout_check_launch("sum_norm");
  }
  // rows that allow no 16-byte accesses: the plain kernel, and with a history the separate steps after it
  float* y2_now = history ? nullptr : y2;
  void* h_now = history ? nullptr : h;
  if (h_now && h_dtype == SPROUT_BF16)
    sprout_launch(sum_norm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, y, gain, x, y2_now, (__nv_bfloat16*)h_now, hidden, eps, alpha);
  else
    sprout_launch(sum_norm_kernel<float>, dim3(rows), dim3(256), 0, stream, y, gain, x, y2_now, (float*)h_now, hidden, eps, alpha);
  if (int code = sprout_check_launch("sum_norm")) return code;
  if (!history) return 0;
  if (int code = sprout_depth_average(history, x, weights, n, plane, stream)) return code;
  if (y2) return sprout_scale_cast(x, y2, h, h_dtype, alpha, plane, stream);
  return 0;
}

SPROUT_API int sprout_polynorm(const void* z, int z_dtype, void* out, int out_dtype, const float* coef, int rows, int width,
                               float eps, cudaStream_t stream) {
  SPROUT_REQUIRE(z && out && coef && rows > 0 && width > 0, "polynorm: null pointer or empty");
  if (z_dtype == SPROUT_F32 && width % 4 == 0 && width <= 8192 && (((uintptr_t)z | (uintptr_t)out) & 15) == 0 &&
      (out_dtype == SPROUT_F32 || out_dtype == SPROUT_BF16)) {
#define POLY_VEC(TO, VEC) sprout_launch(polynorm_vec_kernel<TO, VEC>, dim3(rows), dim3(256), 0, stream, (const float*)z, (TO*)out, coef, width, eps)
#define POLY_PICK(TO) do { if (width <= 1024) POLY_VEC(TO, 1); else if (width <= 2048) POLY_VEC(TO, 2); \
                           else if (width <= 4096) POLY_VEC(TO, 4); else POLY_VEC(TO, 8); } while (0)
    if (out_dtype == SPROUT_BF16) POLY_PICK(__nv_bfloat16); else POLY_PICK(float);
#undef POLY_PICK
#undef POLY_VEC
    return sprout_check_launch("polynorm");
  }
  if (z_dtype == SPROUT_F32 && out_dtype == SPROUT_F32)
    sprout_launch(polynorm_kernel<float, float>, dim3(rows), dim3(256), 0, stream, (const float*)z, (float*)out, coef, width, eps);
  else if (z_dtype == SPROUT_F32 && out_dtype == SPROUT_BF16)
    sprout_launch(polynorm_kernel<float, __nv_bfloat16>, dim3(rows), dim3(256), 0, stream, (const float*)z, (__nv_bfloat16*)out, coef, width, eps);
  else if (z_dtype == SPROUT_BF16 && out_dtype == SPROUT_BF16)
    sprout_launch(polynorm_kernel<__nv_bfloat16, __nv_bfloat16>, dim3(rows), dim3(256), 0, stream, (const __nv_bfloat16*)z, (__nv_bfloat16*)out, coef, width, eps);
  else
    return sprout_fail("polynorm: unsupported dtypes z=%d out=%d", z_dtype, out_dtype);
  return sprout_check_launch("polynorm");
}

SPROUT_API int sprout_latent_kv_append(const float* src, int ld, const float* weight, const int* positions,
                                       const int* seq_of_token, const int* block_table, int table_stride,
                                       const float* cos_table, const float* sin_table, int table_positions,
                                       int rotary_dim, int interleaved, void* cache, int cache_dtype, int tokens,
                                       int rank, int rot, int page_tokens, int num_pages, float eps, int* status,
                                       cudaStream_t stream) {
  SPROUT_REQUIRE(src && weight && positions && seq_of_token && block_table && cache && status, "latent_kv_append: null pointer");
  SPROUT_REQUIRE(tokens > 0 && rank > 0 && rot >= 0 && ld >= rank + rot && page_tokens > 0 && num_pages > 0,
                 "latent_kv_append: sizes do not fit");
  SPROUT_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= rot && (rotary_dim == 0 || (cos_table && sin_table)),
                 "latent_kv_append: the rotated width must be even, at most the key part's width, and come with tables");
  if (cache_dtype == SPROUT_F32)
    sprout_launch(latent_kv_append_kernel<float>, dim3(tokens), dim3(128), 0, stream, src, ld, weight, positions, seq_of_token,
                  block_table, table_stride, cos_table, sin_table, table_positions, rotary_dim, interleaved, (float*)cache,
                  rank, rot, page_tokens, num_pages, eps, status);
  else if (cache_dtype == SPROUT_BF16)
    sprout_launch(latent_kv_append_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, src, ld, weight, positions,
                  seq_of_token, block_table, table_stride, cos_table, sin_table, table_positions, rotary_dim, interleaved,
                  (__nv_bfloat16*)cache, rank, rot, page_tokens, num_pages, eps, status);
  else
    return sprout_fail("latent_kv_append: unknown dtype %d", cache_dtype);
  return sprout_check_launch("latent_kv_append");
}

SPROUT_API int sprout_latent_query_tail(const void* q, void* qlat, int dtype, const int* positions, const float* cos_table,
                                        const float* sin_table, int table_positions, int rotary_dim, int interleaved,
                                        int tokens, int heads, int dim, int rot, int rank, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(q && qlat && positions && status && tokens > 0 && heads > 0 && dim >= 0 && rot >= 0 && rank > 0,
                 "latent_query_tail: null pointer or sizes");
  SPROUT_REQUIRE(rotary_dim >= 0 && rotary_dim % 2 == 0 && rotary_dim <= rot && (rotary_dim == 0 || (cos_table && sin_table)),
                 "latent_query_tail: the rotated width must be even, at most the rotated part's width, and come with tables");
  if (rot == 0) return 0;
  if (dtype == SPROUT_F32)
    sprout_launch(latent_query_tail_kernel<float>, dim3(tokens), dim3(128), 0, stream, (const float*)q, (float*)qlat, positions,
                  cos_table, sin_table, table_positions, rotary_dim, interleaved, heads, dim, rot, rank, status);
  else if (dtype == SPROUT_BF16)
    sprout_launch(latent_query_tail_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, (const __nv_bfloat16*)q,
                  (__nv_bfloat16*)qlat, positions, cos_table, sin_table, table_positions, rotary_dim, interleaved, heads, dim,
                  rot, rank, status);
  else
    return sprout_fail("latent_query_tail: unknown dtype %d", dtype);
  return sprout_check_launch("latent_query_tail");
}

SPROUT_API int sprout_headwise_gemm(const void* a, long long a_row, long long a_head, const void* w, void* out,
                                    long long o_row, long long o_head, int dtype, int rows, int heads, int n, int k,
                                    cudaStream_t stream) {
  SPROUT_REQUIRE(a && w && out && rows > 0 && heads > 0 && n > 0 && k > 0, "headwise_gemm: null pointer or sizes");
  SPROUT_REQUIRE(heads <= 65535 && (rows + HB - 1) / HB <= 65535, "headwise_gemm: too many heads or rows");
  dim3 grid((n + HB - 1) / HB, (rows + HB - 1) / HB, heads);
  if (dtype == SPROUT_F32)
    sprout_launch(headwise_gemm_kernel<float>, grid, dim3(HTHREADS), 0, stream, (const float*)a, a_row, a_head, (const float*)w,
                  (float*)out, o_row, o_head, rows, n, k);
  else if (dtype == SPROUT_BF16 && k % 8 == 0 && a_row % 8 == 0 && a_head % 8 == 0 && n % 2 == 0 && o_row % 2 == 0 && o_head % 2 == 0 &&
           ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)out & 3) == 0)
    // rows that start on 16-byte boundaries and pairs of outputs on 4-byte ones: the tensor-core kernel
    sprout_launch(headwise_gemm_mma_kernel, grid, dim3(128), 0, stream, (const __nv_bfloat16*)a, a_row, a_head,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_row, o_head, rows, n, k);
  else if (dtype == SPROUT_BF16)
    sprout_launch(headwise_gemm_kernel<__nv_bfloat16>, grid, dim3(HTHREADS), 0, stream, (const __nv_bfloat16*)a, a_row, a_head,
                  (const __nv_bfloat16*)w, (__nv_bfloat16*)out, o_row, o_head, rows, n, k);
  else
    return sprout_fail("headwise_gemm: unknown dtype %d", dtype);
  return sprout_check_launch("headwise_gemm");
}

SPROUT_API int sprout_latent_attention_simple(const void* qlat, const void* cache, const int* block_table, int table_stride,
                                              const int* seq_of_token, const int* positions, const float* sink, void* out,
                                              int dtype, int tokens, int heads, int width, int rank, int page_tokens,
                                              int num_pages, float scale, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(qlat && cache && block_table && seq_of_token && positions && out && status, "latent_attention_simple: null pointer");
  SPROUT_REQUIRE(tokens > 0 && heads > 0 && heads <= 65535 && rank > 0 && width >= rank && page_tokens > 0 && num_pages > 0,
                 "latent_attention_simple: sizes do not fit");
  SPROUT_REQUIRE(rank <= MAX_V * CHUNK, "latent_attention_simple: latent size %d above %d", rank, MAX_V * CHUNK);
  const size_t smem = (size_t)(width + (width & 1) + CHUNK + 34) * sizeof(float) + CHUNK * sizeof(long long);
  dim3 grid(tokens, heads);
  if (dtype == SPROUT_F32)
    sprout_launch(latent_attention_simple_kernel<float>, grid, dim3(CHUNK), smem, stream, (const float*)qlat, (const float*)cache,
                  block_table, table_stride, seq_of_token, positions, sink, (float*)out, heads, width, rank, page_tokens,
                  num_pages, scale, status);
  else if (dtype == SPROUT_BF16)
    sprout_launch(latent_attention_simple_kernel<__nv_bfloat16>, grid, dim3(CHUNK), smem, stream, (const __nv_bfloat16*)qlat,
                  (const __nv_bfloat16*)cache, block_table, table_stride, seq_of_token, positions, sink, (__nv_bfloat16*)out,
                  heads, width, rank, page_tokens, num_pages, scale, status);
  else
    return sprout_fail("latent_attention_simple: unknown dtype %d", dtype);
  return sprout_check_launch("latent_attention_simple");
}

SPROUT_API int sprout_depth_average(float* history, float* x, const float* weights, int n, long long plane, cudaStream_t stream) {
  SPROUT_REQUIRE(history && x && weights && n >= 0 && plane > 0, "depth_average: null pointer or sizes");
  if (plane % 4 == 0 && (((uintptr_t)history | (uintptr_t)x) & 15) == 0)
    sprout_launch(depth_average_vec_kernel, dim3(flat_grid(plane / 4, 256)), dim3(256), 0, stream, (float4*)history, (float4*)x, weights,
                  n, plane / 4);
  else
    sprout_launch(depth_average_kernel, dim3(flat_grid(plane, 256)), dim3(256), 0, stream, history, x, weights, n, plane);
  return sprout_check_launch("depth_average");
}

SPROUT_API int sprout_softcap(float* x, float cap, long long count, cudaStream_t stream) {
  SPROUT_REQUIRE(x && count > 0 && cap > 0.f, "softcap: null pointer, no elements or a cap that is not positive");
  sprout_launch(softcap_kernel, dim3(flat_grid(count, 256)), dim3(256), 0, stream, x, cap, count);
  return sprout_check_launch("softcap");
}
