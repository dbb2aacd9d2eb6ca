// Attention whose heads hold one or two score maps over shared values (differential attention), on the
// paged cache, float32 arithmetic.
//
// A key/value head's cache row holds `maps` key vectors of `dim` elements side by side
// ([pages, kv_heads, page_tokens, maps * dim]); its value row has `vdim` elements
// ([pages, kv_heads, page_tokens, vdim]).  A query head has `maps` query vectors; map m of query head h
// scores against map m of key/value head h / (heads / kv_heads): score = scale * q . k, causal, softmax
// per map, a_m = softmax_m V.  The head's output is a_0 - lambda * a_1 (a_0 alone with one map), then,
// with `norm_eps` > 0, divided by its root mean square over vdim, and times `out_scale`.
//
//  * rope_maps_append:          rotates the first `rot` elements of every query and key vector by the
//                               token's position (half-split pairs) and appends keys and values to the cache.
//  * multimap_attention_simple: one block per (token, query head); keys in chunks of 128 aligned to
//                               absolute position with running maxima and sums: what is done for a query
//                               does not depend on how the tokens were cut into steps.
#include "common.cuh"

namespace {

constexpr int CHUNK = 128;

// Row of a token: [q: q_vectors * dim | k: kv_heads * maps * dim | v: kv_heads * vdim] (k and v only when `write`).
template <typename T>
__global__ void __launch_bounds__(128)
rope_maps_append_kernel(T* __restrict__ rows, int row_stride, const int* __restrict__ positions,
                        const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int table_stride,
                        const float* __restrict__ cos_table, const float* __restrict__ sin_table, int max_positions,
                        T* __restrict__ k_cache, T* __restrict__ v_cache, int q_vectors, int kv_heads, int maps, int dim,
                        int rot, int vdim, int page_tokens, int num_pages, int write, int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  T* row = rows + (size_t)t * row_stride;
  const int half = rot / 2;
  const bool turn = rot > 0 && pos >= 0 && pos < max_positions;
  if (rot > 0 && !turn && threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_POSITION);
  const float* cs = cos_table + (size_t)(turn ? pos : 0) * half;
  const float* sn = sin_table + (size_t)(turn ? pos : 0) * half;
  // queries: in place
  if (turn) {
    for (int i = threadIdx.x; i < q_vectors * half; i += blockDim.x) {
      T* vec = row + (size_t)(i / half) * dim;
      const int d = i % half;
      const float u = to_float(vec[d]), v = to_float(vec[d + half]);
      const float c = cs[d], s = sn[d];
      vec[d] = from_float<T>(u * c - v * s);
      vec[d + half] = from_float<T>(v * c + u * s);
    }
  }
  if (!write) return;
  const int page = block_table[(size_t)seq_of_token[t] * table_stride + pos / page_tokens];
  if (page < 0 || page >= num_pages) {
    if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  const T* krow = row + (size_t)q_vectors * dim;
  const T* vrow = krow + (size_t)kv_heads * maps * dim;
  const int kw = maps * dim;
  for (int i = threadIdx.x; i < kv_heads * kw; i += blockDim.x) {
    const int g = i / kw, e = i % kw, d = e % dim;
    float value = to_float(krow[i]);
    if (turn && d < rot) {
      const int j = d < half ? d : d - half;
      const float other = to_float(krow[i + (d < half ? half : -half)]);
      value = d < half ? value * cs[j] - other * sn[j] : value * cs[j] + other * sn[j];
    }
    k_cache[(((size_t)page * kv_heads + g) * page_tokens + pos % page_tokens) * kw + e] = from_float<T>(value);
  }
  for (int i = threadIdx.x; i < kv_heads * vdim; i += blockDim.x) {
    const int g = i / vdim, e = i % vdim;
    v_cache[(((size_t)page * kv_heads + g) * page_tokens + pos % page_tokens) * vdim + e] = vrow[i];
  }
}

template <typename T, int MAPS>
__global__ void __launch_bounds__(CHUNK)
multimap_attention_simple_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ k_cache,
                                 const T* __restrict__ v_cache, const int* __restrict__ block_table, int table_stride,
                                 const int* __restrict__ seq_of_token, const int* __restrict__ positions,
                                 T* __restrict__ out, int out_stride, int heads, int kv_heads, int dim, int vdim,
                                 int page_tokens, int num_pages, float scale, float lambda, float norm_eps,
                                 float out_scale, int* status) {
  extern __shared__ float smem[];
  float* qs = smem;                                   // MAPS * dim
  float* probs = qs + MAPS * dim;                     // MAPS * CHUNK
  float* scratch = probs + MAPS * CHUNK;              // 34
  long long* row_index = (long long*)(scratch + 34 + ((MAPS * dim) & 1));   // CHUNK, 8-byte aligned

  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int g = h / (heads / kv_heads);
  const int pos = positions[t];
  const int* table = block_table + (size_t)seq_of_token[t] * table_stride;
  const int kw = MAPS * dim;
  for (int d = tid; d < kw; d += CHUNK) qs[d] = to_float(q[(size_t)t * q_stride + (size_t)h * kw + d]);
  __syncthreads();

  float m_run[MAPS], l_run[MAPS], acc[MAPS][2];
#pragma unroll
  for (int m = 0; m < MAPS; m++) {
    m_run[m] = -INFINITY;
    l_run[m] = 0.f;
    acc[m][0] = acc[m][1] = 0.f;
  }
  for (int base = 0; base <= pos; base += CHUNK) {
    const int p = base + tid;
    bool valid = p <= pos;
    long long index = -1;
    if (valid) {
      const int page = table[p / page_tokens];
      if (page < 0 || page >= num_pages) {
        atomicOr(status, SPROUT_STATUS_BAD_PAGE);
        valid = false;
      } else {
        index = ((long long)page * kv_heads + g) * page_tokens + (p % page_tokens);
      }
    }
    float s[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      s[m] = -INFINITY;
      if (valid) {
        const T* key = k_cache + index * kw + m * dim;
        float dot = 0.f;
        for (int d = 0; d < dim; d++) dot = fmaf(qs[m * dim + d], to_float(key[d]), dot);
        s[m] = dot * scale;
      }
    }
    row_index[tid] = index;
    float alpha[MAPS];
#pragma unroll
    for (int m = 0; m < MAPS; m++) {
      const float m_new = fmaxf(m_run[m], block_max(s[m], scratch));
      const float e = valid ? expf(s[m] - m_new) : 0.f;
      probs[m * CHUNK + tid] = e;
      const float c_sum = block_sum(e, scratch);
      alpha[m] = (m_run[m] == -INFINITY) ? 0.f : expf(m_run[m] - m_new);
      l_run[m] = l_run[m] * alpha[m] + c_sum;
      m_run[m] = m_new;
    }
    __syncthreads();
    const int count = min(CHUNK, pos - base + 1);
#pragma unroll
    for (int part = 0; part < 2; part++) {
      const int e = tid + part * CHUNK;
      if (e < vdim) {
#pragma unroll
        for (int m = 0; m < MAPS; m++) acc[m][part] *= alpha[m];
        for (int j = 0; j < count; j++) {
          const long long r = row_index[j];
          if (r < 0) continue;
          const float v = to_float(v_cache[r * vdim + e]);
#pragma unroll
          for (int m = 0; m < MAPS; m++) acc[m][part] = fmaf(probs[m * CHUNK + j], v, acc[m][part]);
        }
      }
    }
    __syncthreads();
  }
  float o[2];
  float squares = 0.f;
#pragma unroll
  for (int part = 0; part < 2; part++) {
    o[part] = acc[0][part] / l_run[0];
    if (MAPS == 2) o[part] -= lambda * (acc[MAPS - 1][part] / l_run[MAPS - 1]);
    if (tid + part * CHUNK < vdim) squares = fmaf(o[part], o[part], squares);
  }
  float factor = out_scale;
  if (norm_eps > 0.f) factor *= 1.0f / sqrtf(block_sum(squares, scratch) / (float)vdim + norm_eps);
  T* dst = out + (size_t)t * out_stride + (size_t)h * vdim;
#pragma unroll
  for (int part = 0; part < 2; part++)
    if (tid + part * CHUNK < vdim) dst[tid + part * CHUNK] = from_float<T>(o[part] * factor);
}

}  // namespace

SPROUT_API int sprout_rope_maps_append(void* rows, int row_stride, int dtype, const int* positions, const int* seq_of_token,
                                       const int* block_table, int table_stride, const float* cos_table,
                                       const float* sin_table, int max_positions, void* k_cache, void* v_cache, int tokens,
                                       int q_vectors, int kv_heads, int maps, int dim, int rot, int vdim, int page_tokens,
                                       int num_pages, int write, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(rows && positions && status && tokens > 0 && q_vectors > 0 && dim > 0 && maps > 0, "rope_maps_append: bad arguments");
  SPROUT_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= dim, "rope_maps_append: the rotated width must be even and at most dim");
  SPROUT_REQUIRE(rot == 0 || (cos_table && sin_table && max_positions > 0), "rope_maps_append: tables are missing");
  SPROUT_REQUIRE(!write || (k_cache && v_cache && seq_of_token && block_table && kv_heads > 0 && vdim > 0 && page_tokens > 0 &&
                            num_pages > 0), "rope_maps_append: the cache is missing");
  const int need = q_vectors * dim + (write ? kv_heads * (maps * dim + vdim) : 0);
  SPROUT_REQUIRE(row_stride >= need, "rope_maps_append: rows of %d elements, %d needed", row_stride, need);
  if (dtype == SPROUT_F32)
    sprout_launch(rope_maps_append_kernel<float>, dim3(tokens), dim3(128), 0, stream, (float*)rows, row_stride, positions,
                  seq_of_token, block_table, table_stride, cos_table, sin_table, max_positions, (float*)k_cache,
                  (float*)v_cache, q_vectors, kv_heads, maps, dim, rot, vdim, page_tokens, num_pages, write, status);
  else if (dtype == SPROUT_BF16)
    sprout_launch(rope_maps_append_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, (__nv_bfloat16*)rows, row_stride,
                  positions, seq_of_token, block_table, table_stride, cos_table, sin_table, max_positions,
                  (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, q_vectors, kv_heads, maps, dim, rot, vdim, page_tokens,
                  num_pages, write, status);
  else
    return sprout_fail("rope_maps_append: unknown dtype %d", dtype);
  return sprout_check_launch("rope_maps_append");
}

SPROUT_API int sprout_multimap_attention_simple(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                                                const int* block_table, int table_stride, const int* seq_of_token,
                                                const int* positions, void* out, int out_stride, int dtype, int tokens,
                                                int heads, int kv_heads, int maps, int dim, int vdim, int page_tokens,
                                                int num_pages, float scale, float lambda, float norm_eps, float out_scale,
                                                int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(q && k_cache && v_cache && block_table && seq_of_token && positions && out && status, "multimap_attention: null pointer");
  SPROUT_REQUIRE(tokens > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && page_tokens > 0 && num_pages > 0,
                 "multimap_attention: bad sizes");
  SPROUT_REQUIRE(maps == 1 || maps == 2, "multimap_attention: one or two maps per head (got %d)", maps);
  SPROUT_REQUIRE(dim > 0 && vdim > 0 && vdim <= 2 * CHUNK, "multimap_attention: value rows of up to %d elements (got %d)", 2 * CHUNK, vdim);
  SPROUT_REQUIRE(heads <= 65535, "multimap_attention: too many heads");
  const size_t smem = (size_t)(maps * dim + maps * CHUNK + 36) * sizeof(float) + CHUNK * sizeof(long long);
  SPROUT_REQUIRE(smem <= 48 * 1024, "multimap_attention: key vectors too long (%d)", dim);
  dim3 grid(tokens, heads);
#define LAUNCH(T, M)                                                                                                      \
  sprout_launch(multimap_attention_simple_kernel<T, M>, grid, dim3(CHUNK), smem, stream, (const T*)q, q_stride,           \
                (const T*)k_cache, (const T*)v_cache, block_table, table_stride, seq_of_token, positions, (T*)out,        \
                out_stride, heads, kv_heads, dim, vdim, page_tokens, num_pages, scale, lambda, norm_eps, out_scale, status)
  if (dtype == SPROUT_F32) {
    if (maps == 1) LAUNCH(float, 1); else LAUNCH(float, 2);
  } else if (dtype == SPROUT_BF16) {
    if (maps == 1) LAUNCH(__nv_bfloat16, 1); else LAUNCH(__nv_bfloat16, 2);
  } else {
    return sprout_fail("multimap_attention: unknown dtype %d", dtype);
  }
#undef LAUNCH
  return sprout_check_launch("multimap_attention_simple");
}
