// Linear attention with a per-head decay and a state per request ("lightning attention"):
//   S_t = decay_h * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t        (S: [dim, vdim] per head, float32)
// with q, k, v = act(projection) (act = silu, or none).  The state of a request lives in a slot of a
// buffer [slots, heads, dim, vdim]; a step reads it, runs the request's tokens of this step and writes it
// back, so a prompt may be cut anywhere.
//
//  * decay_scan:  one block per (request, head, block of value columns), token by token in float32: thread j
//                 owns column j of the state; the order of operations per element is the tokens' order, so the
//                 result does not depend on the cutting or on the batch.
//  * decay_chunks: bfloat16 prompts on tensor cores (`mma.sync.m16n8k16`), 64 tokens at a time: with n tokens in the
//                 chunk and S the state before it,
//                   o_i = sum_{j <= i} decay^(i-j) (q_i . k_j) v_j + decay^(i+1) q_i^T S,
//                   S  <- decay^n S + sum_j (decay^(n-1-j) k_j) v_j^T.
//                 A CTA owns (request, head, 64 value columns) and keeps its part of S in accumulator registers
//                 (float32) from chunk to chunk.  What enters the recurrence stays 32-bit in effect: the decayed keys
//                 and the state read by the queries go to the tensor cores as two bfloat16 terms each (value = high +
//                 low), so their rounding is 2^-17, not 2^-9; the decay powers are float32.  Two forms: a CTA walking its
//                 request's chunks in order, and (the default) all chunks at once in three launches: every chunk's own
//                 sum of decayed key-value products, a scan over each request's chunks, every chunk's outputs.
// A token's row holds [q: heads * dim | k: heads * dim | v: heads * vdim | ...] as the projection left it.
#include "attention_bf16.cuh"

using namespace sprout_attn;

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__device__ __forceinline__ float activate(T raw, int act) {
  const float z = to_float(raw);
  // the activation's result is rounded to the projection's type: it is what a product in that type would read
  return act ? to_float(from_float<T>(silu_f(z))) : z;
}

template <typename T>
__global__ void __launch_bounds__(256)
decay_scan_kernel(const T* __restrict__ rows, int row_stride, const int* __restrict__ q_start,
                  const int* __restrict__ state_slots, float* __restrict__ state, int num_slots,
                  const float* __restrict__ decay, float* __restrict__ out, int heads, int dim, int vdim, int act,
                  int* status) {
  extern __shared__ float smem[];
  float* S = smem;                          // dim * cols
  float* qk = S + (size_t)dim * blockDim.x; // 2 * dim
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y, cols = blockDim.x;
  const int col = blockIdx.z * cols + threadIdx.x;
  const bool live = col < vdim;
  const int slot = state_slots[r];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  float* mine = state + (((size_t)slot * heads + h) * dim) * vdim;
  if (live)
    for (int i = 0; i < dim; i++) S[i * cols + threadIdx.x] = mine[(size_t)i * vdim + col];
  const float lam = decay[h];
  const int first = q_start[r], last = q_start[r + 1];
  for (int t = first; t < last; t++) {
    const T* row = rows + (size_t)t * row_stride;
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * dim; i += cols)
      qk[i] = activate(row[(size_t)(i < dim ? 0 : heads * dim) + (size_t)h * dim + (i < dim ? i : i - dim)], act);
    __syncthreads();
    if (!live) continue;
    const float v = activate(row[(size_t)2 * heads * dim + (size_t)h * vdim + col], act);
    float o = 0.f;
    for (int i = 0; i < dim; i++) {
      const float s = fmaf(lam, S[i * cols + threadIdx.x], qk[dim + i] * v);
      S[i * cols + threadIdx.x] = s;
      o = fmaf(s, qk[i], o);
    }
    out[(size_t)t * heads * vdim + (size_t)h * vdim + col] = o;
  }
  if (live)
    for (int i = 0; i < dim; i++) mine[(size_t)i * vdim + col] = S[i * cols + threadIdx.x];
}


// ------------------------------------------------------------------------------------------ tensor cores
constexpr int DC = 64, DVB = 64, DC_THREADS = 128;     // tokens per chunk, value columns per CTA

// q, k, v of a row in place: act(x) as bfloat16 holds it (the chunked kernels then copy tiles as they are); 8 elements a thread
__global__ void silu_rows_kernel(__nv_bfloat16* __restrict__ rows, int row_stride, int width8, long long count8) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count8; i += (long long)gridDim.x * blockDim.x) {
    uint4* at = (uint4*)(rows + (i / width8) * row_stride + (i % width8) * 8);
    uint4 v = *at;
    __nv_bfloat162* pair = (__nv_bfloat162*)&v;
#pragma unroll
    for (int e = 0; e < 4; e++) pair[e] = __floats2bfloat162_rn(silu_f(__low2float(pair[e])), silu_f(__high2float(pair[e])));
    *at = v;
  }
}

template <int DIM>
__global__ void __launch_bounds__(DC_THREADS)
decay_chunks_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, const int* __restrict__ q_start,
                    const int* __restrict__ state_slots, float* __restrict__ state, int num_slots,
                    const float* __restrict__ decay, float* __restrict__ out, int heads, int vdim, int* status) {
  constexpr int QS = DIM + 8, VS = DVB + 8, MT = DIM / 64;        // a warp owns DIM / 4 rows of the state: MT tiles of 16
  constexpr int QCH = DIM / 8, VCH = DVB / 8;
  extern __shared__ __align__(16) unsigned char dc_smem[];
  __nv_bfloat16* sQ = (__nv_bfloat16*)dc_smem;                    // 2 x DC x QS
  __nv_bfloat16* sK = sQ + 2 * DC * QS;                           // 2 x DC x QS
  __nv_bfloat16* sKh = sK + 2 * DC * QS;                          // decayed keys, high and low terms
  __nv_bfloat16* sKl = sKh + DC * QS;
  __nv_bfloat16* sV = sKl + DC * QS;                              // 2 x DC x VS
  __nv_bfloat16* sSh = sV + 2 * DC * VS;                          // DIM x VS: the state, high and low terms
  __nv_bfloat16* sSl = sSh + DIM * VS;
  __shared__ float power[DC + 1];                                 // decay^e
  pdl_launch_dependents();
  const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DVB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gr = lane >> 2, qc = lane & 3;
  if (tid <= DC) power[tid] = exp2f((float)tid * log2f(decay[h]));
  pdl_wait();
  const int slot = state_slots[r];
  if (slot < 0 || slot >= num_slots) {
    if (tid == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  float* mine = state + (((size_t)slot * heads + h) * DIM) * vdim;
  float S[MT][DVB / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; mt++)
#pragma unroll
    for (int nt = 0; nt < DVB / 8; nt++)
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const int row = warp * (DIM / 4) + mt * 16 + gr + (c >> 1) * 8, col = col0 + nt * 8 + qc * 2 + (c & 1);
        S[mt][nt][c] = col < vdim ? mine[(size_t)row * vdim + col] : 0.f;
      }
  const int first = q_start[r], last = q_start[r + 1];
  auto load = [&](int buf, int t0) {
    const int n = min(DC, last - t0);
    for (int idx = tid; idx < DC * QCH; idx += DC_THREADS) {
      const int j = idx / QCH, c = (idx % QCH) * 8;
      __nv_bfloat16* dq = sQ + (buf * DC + j) * QS + c;
      __nv_bfloat16* dk = sK + (buf * DC + j) * QS + c;
      if (j < n) {
        const __nv_bfloat16* src = rows + (size_t)(t0 + j) * row_stride + (size_t)h * DIM + c;
        cp_async16(dq, src);
        cp_async16(dk, src + (size_t)heads * DIM);
      } else {
        *(uint4*)dq = make_uint4(0, 0, 0, 0);
        *(uint4*)dk = make_uint4(0, 0, 0, 0);
      }
    }
    for (int idx = tid; idx < DC * VCH; idx += DC_THREADS) {
      const int j = idx / VCH, c = (idx % VCH) * 8;
      __nv_bfloat16* dv = sV + (buf * DC + j) * VS + c;
      if (j < n && col0 + c < vdim) cp_async16(dv, rows + (size_t)(t0 + j) * row_stride + (size_t)2 * heads * DIM + (size_t)h * vdim + col0 + c);
      else *(uint4*)dv = make_uint4(0, 0, 0, 0);
    }
  };
  if (first < last) load(0, first);
  cp_async_commit();
  int buf = 0;
  for (int t0 = first; t0 < last; t0 += DC, buf ^= 1) {
    const int n = min(DC, last - t0);
    cp_async_wait<0>();
    __syncthreads();                                   // the chunk has landed; the chunk before is done with shared memory
    if (t0 + DC < last) load(buf ^ 1, t0 + DC);
    cp_async_commit();
    const __nv_bfloat16* tQ = sQ + buf * DC * QS;
    const __nv_bfloat16* tK = sK + buf * DC * QS;
    const __nv_bfloat16* tV = sV + buf * DC * VS;
    // the decayed keys in two terms
    for (int idx = tid; idx < DC * QCH; idx += DC_THREADS) {
      const int j = idx / QCH, c = (idx % QCH) * 8;
      const float w = j < n ? power[n - 1 - j] : 0.f;
      const uint4 raw = *(const uint4*)(tK + j * QS + c);
      const __nv_bfloat162* pair = (const __nv_bfloat162*)&raw;
      uint4 hi, lo;
      __nv_bfloat162* ph = (__nv_bfloat162*)&hi;
      __nv_bfloat162* pl = (__nv_bfloat162*)&lo;
#pragma unroll
      for (int e = 0; e < 4; e++) {
        const float a = __low2float(pair[e]) * w, b = __high2float(pair[e]) * w;
        ph[e] = __floats2bfloat162_rn(a, b);
        pl[e] = __floats2bfloat162_rn(a - __low2float(ph[e]), b - __high2float(ph[e]));
      }
      *(uint4*)(sKh + j * QS + c) = hi;
      *(uint4*)(sKl + j * QS + c) = lo;
    }
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
      for (int nt = 0; nt < DVB / 8; nt++)
#pragma unroll
        for (int half = 0; half < 2; half++) {
          const int row = warp * (DIM / 4) + mt * 16 + gr + half * 8, col = nt * 8 + qc * 2;
          const float a = S[mt][nt][half * 2], b = S[mt][nt][half * 2 + 1];
          const __nv_bfloat162 hi = __floats2bfloat162_rn(a, b);
          *(__nv_bfloat162*)(sSh + row * VS + col) = hi;
          *(__nv_bfloat162*)(sSl + row * VS + col) = __floats2bfloat162_rn(a - __low2float(hi), b - __high2float(hi));
        }
    __syncthreads();

    // scores of the chunk: rows 16 warp .. 16 warp + 15 against its 64 keys
    float s[DC / 8][4];
#pragma unroll
    for (int i = 0; i < DC / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
    float o[DVB / 8][4];
#pragma unroll
    for (int i = 0; i < DVB / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DIM / 16; kk++) {
      uint32_t a[4];
      ldmatrix_x4(a, tQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int n2 = 0; n2 < DC / 16; n2++) {
        uint32_t b[4];
        ldmatrix_x4(b, tK + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * QS + kk * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * n2], a, b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
      }
      // the same query fragment against the state before the chunk (two terms)
#pragma unroll
      for (int d2 = 0; d2 < DVB / 16; d2++) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, sSh + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * d2], a, b[0], b[1]);
        mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
        ldmatrix_x4_trans(b, sSl + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * d2], a, b[0], b[1]);
        mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
      }
    }
    const int i0 = warp * 16 + gr, i1 = i0 + 8;        // the thread's two rows (tokens of the chunk)
    const float carry0 = power[i0 + 1], carry1 = power[i1 + 1];
#pragma unroll
    for (int i = 0; i < DVB / 8; i++) { o[i][0] *= carry0; o[i][1] *= carry0; o[i][2] *= carry1; o[i][3] *= carry1; }
#pragma unroll
    for (int i = 0; i < DC / 8; i++) {
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const int j = i * 8 + qc * 2 + c;
        s[i][c] = j <= i0 ? s[i][c] * power[i0 - j] : 0.f;
        s[i][2 + c] = j <= i1 ? s[i][2 + c] * power[i1 - j] : 0.f;
      }
    }
#pragma unroll
    for (int kk = 0; kk < DC / 16; kk++) {
      uint32_t a[4];
      a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
      for (int d2 = 0; d2 < DVB / 16; d2++) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, tV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * d2], a, b[0], b[1]);
        mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
      }
    }
#pragma unroll
    for (int half = 0; half < 2; half++) {
      const int i = half ? i1 : i0;
      if (i >= n) continue;
      float* dst = out + (size_t)(t0 + i) * heads * vdim + (size_t)h * vdim + col0;
#pragma unroll
      for (int nt = 0; nt < DVB / 8; nt++) {
        const int col = nt * 8 + qc * 2;
        if (col0 + col < vdim) *(float2*)(dst + col) = make_float2(o[nt][half * 2], o[nt][half * 2 + 1]);
      }
    }

    // the state after the chunk: decay^n S + (decayed keys)^T V, the keys' two terms one after the other
    const float shrink = power[n];
#pragma unroll
    for (int mt = 0; mt < MT; mt++) {
#pragma unroll
      for (int nt = 0; nt < DVB / 8; nt++)
#pragma unroll
        for (int c = 0; c < 4; c++) S[mt][nt][c] *= shrink;
#pragma unroll
      for (int kk = 0; kk < DC / 16; kk++) {
        // A = K^T: element (m = key dimension, k = token) lies at [token][dimension], so the 8x8 blocks are read transposed
        const int krow = kk * 16 + (lane & 7) + (lane >> 4) * 8, kcol = warp * (DIM / 4) + mt * 16 + ((lane >> 3) & 1) * 8;
        uint32_t ah[4], al[4];
        ldmatrix_x4_trans(ah, sKh + krow * QS + kcol);
        ldmatrix_x4_trans(al, sKl + krow * QS + kcol);
#pragma unroll
        for (int d2 = 0; d2 < DVB / 16; d2++) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, tV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
          mma_bf16(S[mt][2 * d2], ah, b[0], b[1]);
          mma_bf16(S[mt][2 * d2 + 1], ah, b[2], b[3]);
          mma_bf16(S[mt][2 * d2], al, b[0], b[1]);
          mma_bf16(S[mt][2 * d2 + 1], al, b[2], b[3]);
        }
      }
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int mt = 0; mt < MT; mt++)
#pragma unroll
    for (int nt = 0; nt < DVB / 8; nt++)
#pragma unroll
      for (int c = 0; c < 4; c++) {
        const int row = warp * (DIM / 4) + mt * 16 + gr + (c >> 1) * 8, col = col0 + nt * 8 + qc * 2 + (c & 1);
        if (col < vdim) mine[(size_t)row * vdim + col] = S[mt][nt][c];
      }
}

// ---- the same in three launches, every chunk at once: (1) each chunk's own sum of decayed key-value products,
// (2) per request a scan over its chunks that leaves the state before each chunk in the sums' place and the final state
// in the slot, (3) each chunk's outputs from its tokens and the state before it.
__device__ __forceinline__ bool find_chunk(const int* q_start, int requests, int chunk, int& r, int& t0, int& n) {
  for (r = 0; r < requests; r++) {
    const int first = q_start[r], count = q_start[r + 1] - first, chunks = (count + DC - 1) / DC;
    if (chunk < chunks) {
      t0 = first + chunk * DC;
      n = min(DC, count - chunk * DC);
      return true;
    }
    chunk -= chunks;
  }
  return false;
}

template <int DIM>
__global__ void __launch_bounds__(DC_THREADS)
decay_chunk_sums_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, const int* __restrict__ q_start, int requests,
                        const float* __restrict__ decay, float* __restrict__ sums, int heads, int vdim) {
  constexpr int QS = DIM + 8, VS = DVB + 8, MT = DIM / 64, QCH = DIM / 8, VCH = DVB / 8;
  extern __shared__ __align__(16) unsigned char dc_smem[];
  __nv_bfloat16* sK = (__nv_bfloat16*)dc_smem;                    // DC x QS
  __nv_bfloat16* sKh = sK + DC * QS;
  __nv_bfloat16* sKl = sKh + DC * QS;
  __nv_bfloat16* sV = sKl + DC * QS;                              // DC x VS
  __shared__ float power[DC + 1];
  pdl_launch_dependents();
  const int h = blockIdx.y, col0 = blockIdx.z * DVB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gr = lane >> 2, qc = lane & 3;
  if (tid <= DC) power[tid] = exp2f((float)tid * log2f(decay[h]));
  pdl_wait();
  int r, t0, n;
  if (!find_chunk(q_start, requests, blockIdx.x, r, t0, n)) return;
  for (int idx = tid; idx < DC * QCH; idx += DC_THREADS) {
    const int j = idx / QCH, c = (idx % QCH) * 8;
    if (j < n) cp_async16(sK + j * QS + c, rows + (size_t)(t0 + j) * row_stride + (size_t)heads * DIM + (size_t)h * DIM + c);
    else *(uint4*)(sK + j * QS + c) = make_uint4(0, 0, 0, 0);
  }
  for (int idx = tid; idx < DC * VCH; idx += DC_THREADS) {
    const int j = idx / VCH, c = (idx % VCH) * 8;
    if (j < n && col0 + c < vdim) cp_async16(sV + j * VS + c, rows + (size_t)(t0 + j) * row_stride + (size_t)2 * heads * DIM + (size_t)h * vdim + col0 + c);
    else *(uint4*)(sV + j * VS + c) = make_uint4(0, 0, 0, 0);
  }
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  for (int idx = tid; idx < DC * QCH; idx += DC_THREADS) {
    const int j = idx / QCH, c = (idx % QCH) * 8;
    const float w = j < n ? power[n - 1 - j] : 0.f;
    const uint4 raw = *(const uint4*)(sK + j * QS + c);
    const __nv_bfloat162* pair = (const __nv_bfloat162*)&raw;
    uint4 hi, lo;
    __nv_bfloat162* ph = (__nv_bfloat162*)&hi;
    __nv_bfloat162* pl = (__nv_bfloat162*)&lo;
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const float a = __low2float(pair[e]) * w, b = __high2float(pair[e]) * w;
      ph[e] = __floats2bfloat162_rn(a, b);
      pl[e] = __floats2bfloat162_rn(a - __low2float(ph[e]), b - __high2float(ph[e]));
    }
    *(uint4*)(sKh + j * QS + c) = hi;
    *(uint4*)(sKl + j * QS + c) = lo;
  }
  __syncthreads();
  float U[MT][DVB / 8][4];
#pragma unroll
  for (int mt = 0; mt < MT; mt++) {
#pragma unroll
    for (int nt = 0; nt < DVB / 8; nt++) U[mt][nt][0] = U[mt][nt][1] = U[mt][nt][2] = U[mt][nt][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < DC / 16; kk++) {
      const int krow = kk * 16 + (lane & 7) + (lane >> 4) * 8, kcol = warp * (DIM / 4) + mt * 16 + ((lane >> 3) & 1) * 8;
      uint32_t ah[4], al[4];
      ldmatrix_x4_trans(ah, sKh + krow * QS + kcol);
      ldmatrix_x4_trans(al, sKl + krow * QS + kcol);
#pragma unroll
      for (int d2 = 0; d2 < DVB / 16; d2++) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
        mma_bf16(U[mt][2 * d2], ah, b[0], b[1]);
        mma_bf16(U[mt][2 * d2 + 1], ah, b[2], b[3]);
        mma_bf16(U[mt][2 * d2], al, b[0], b[1]);
        mma_bf16(U[mt][2 * d2 + 1], al, b[2], b[3]);
      }
    }
  }
  float* dst = sums + ((size_t)blockIdx.x * heads + h) * DIM * vdim;
#pragma unroll
  for (int mt = 0; mt < MT; mt++)
#pragma unroll
    for (int nt = 0; nt < DVB / 8; nt++)
#pragma unroll
      for (int half = 0; half < 2; half++) {
        const int row = warp * (DIM / 4) + mt * 16 + gr + half * 8, col = col0 + nt * 8 + qc * 2;
        if (col < vdim) *(float2*)(dst + (size_t)row * vdim + col) = make_float2(U[mt][nt][half * 2], U[mt][nt][half * 2 + 1]);
      }
}

// grid (requests, heads, blocks over dim * vdim): S walks the request's chunks; sums[c] becomes the state before chunk c.
__global__ void __launch_bounds__(256)
decay_chunk_scan_kernel(const int* __restrict__ q_start, const int* __restrict__ state_slots, float* __restrict__ state,
                        int num_slots, const float* __restrict__ decay, float* __restrict__ sums, int heads, int plane,
                        int* status) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y;
  const int slot = state_slots[r];
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0 && blockIdx.z == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  int chunk0 = 0;
  for (int i = 0; i < r; i++) chunk0 += (q_start[i + 1] - q_start[i] + DC - 1) / DC;
  const int count = q_start[r + 1] - q_start[r], chunks = (count + DC - 1) / DC;
  const float log_lam = log2f(decay[h]);
  const float full = exp2f((float)DC * log_lam), tail = exp2f((float)(count - (chunks - 1) * DC) * log_lam);
  float* mine = state + ((size_t)slot * heads + h) * plane;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;             // one element of the state per thread
  if (e >= plane) return;
  float S = mine[e];
  float* at = sums + ((size_t)chunk0 * heads + h) * plane + e;
  const size_t step = (size_t)heads * plane;
  for (int c0 = 0; c0 < chunks; c0 += 8) {                          // eight chunks' sums are fetched before the first is used
    float u[8];
#pragma unroll
    for (int i = 0; i < 8; i++) u[i] = c0 + i < chunks ? at[(size_t)(c0 + i) * step] : 0.f;
#pragma unroll
    for (int i = 0; i < 8; i++) {
      if (c0 + i >= chunks) break;
      at[(size_t)(c0 + i) * step] = S;
      S = fmaf(c0 + i == chunks - 1 ? tail : full, S, u[i]);
    }
  }
  mine[e] = S;
}

template <int DIM>
__global__ void __launch_bounds__(DC_THREADS)
decay_chunk_outputs_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, const int* __restrict__ q_start, int requests,
                           const float* __restrict__ decay, const float* __restrict__ before, float* __restrict__ out,
                           int heads, int vdim) {
  constexpr int QS = DIM + 8, VS = DVB + 8, QCH = DIM / 8, VCH = DVB / 8;
  extern __shared__ __align__(16) unsigned char dc_smem[];
  __nv_bfloat16* sQ = (__nv_bfloat16*)dc_smem;                    // DC x QS
  __nv_bfloat16* sK = sQ + DC * QS;
  __nv_bfloat16* sV = sK + DC * QS;                               // DC x VS
  __nv_bfloat16* sSh = sV + DC * VS;                              // DIM x VS
  __nv_bfloat16* sSl = sSh + DIM * VS;
  __shared__ float power[DC + 1];
  pdl_launch_dependents();
  const int h = blockIdx.y, col0 = blockIdx.z * DVB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gr = lane >> 2, qc = lane & 3;
  if (tid <= DC) power[tid] = exp2f((float)tid * log2f(decay[h]));
  pdl_wait();
  int r, t0, n;
  if (!find_chunk(q_start, requests, blockIdx.x, r, t0, n)) return;
  for (int idx = tid; idx < DC * QCH; idx += DC_THREADS) {
    const int j = idx / QCH, c = (idx % QCH) * 8;
    if (j < n) {
      const __nv_bfloat16* src = rows + (size_t)(t0 + j) * row_stride + (size_t)h * DIM + c;
      cp_async16(sQ + j * QS + c, src);
      cp_async16(sK + j * QS + c, src + (size_t)heads * DIM);
    } else {
      *(uint4*)(sQ + j * QS + c) = make_uint4(0, 0, 0, 0);
      *(uint4*)(sK + j * QS + c) = make_uint4(0, 0, 0, 0);
    }
  }
  for (int idx = tid; idx < DC * VCH; idx += DC_THREADS) {
    const int j = idx / VCH, c = (idx % VCH) * 8;
    if (j < n && col0 + c < vdim) cp_async16(sV + j * VS + c, rows + (size_t)(t0 + j) * row_stride + (size_t)2 * heads * DIM + (size_t)h * vdim + col0 + c);
    else *(uint4*)(sV + j * VS + c) = make_uint4(0, 0, 0, 0);
  }
  cp_async_commit();
  // the state before the chunk, as two bfloat16 terms
  const float* S = before + ((size_t)blockIdx.x * heads + h) * DIM * vdim;
  for (int idx = tid; idx < DIM * (DVB / 2); idx += DC_THREADS) {
    const int row = idx / (DVB / 2), col = (idx % (DVB / 2)) * 2;
    float a = 0.f, b = 0.f;
    if (col0 + col < vdim) {
      const float2 v = *(const float2*)(S + (size_t)row * vdim + col0 + col);
      a = v.x; b = v.y;
    }
    const __nv_bfloat162 hi = __floats2bfloat162_rn(a, b);
    *(__nv_bfloat162*)(sSh + row * VS + col) = hi;
    *(__nv_bfloat162*)(sSl + row * VS + col) = __floats2bfloat162_rn(a - __low2float(hi), b - __high2float(hi));
  }
  cp_async_wait<0>();
  __syncthreads();
  float s[DC / 8][4];
#pragma unroll
  for (int i = 0; i < DC / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
  float o[DVB / 8][4];
#pragma unroll
  for (int i = 0; i < DVB / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
#pragma unroll
  for (int kk = 0; kk < DIM / 16; kk++) {
    uint32_t a[4];
    ldmatrix_x4(a, sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int n2 = 0; n2 < DC / 16; n2++) {
      uint32_t b[4];
      ldmatrix_x4(b, sK + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * QS + kk * 16 + ((lane >> 3) & 1) * 8);
      mma_bf16(s[2 * n2], a, b[0], b[1]);
      mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
    }
#pragma unroll
    for (int d2 = 0; d2 < DVB / 16; d2++) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, sSh + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
      mma_bf16(o[2 * d2], a, b[0], b[1]);
      mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
      ldmatrix_x4_trans(b, sSl + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
      mma_bf16(o[2 * d2], a, b[0], b[1]);
      mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
    }
  }
  const int i0 = warp * 16 + gr, i1 = i0 + 8;
  const float carry0 = power[i0 + 1], carry1 = power[i1 + 1];
#pragma unroll
  for (int i = 0; i < DVB / 8; i++) { o[i][0] *= carry0; o[i][1] *= carry0; o[i][2] *= carry1; o[i][3] *= carry1; }
#pragma unroll
  for (int i = 0; i < DC / 8; i++) {
#pragma unroll
    for (int c = 0; c < 2; c++) {
      const int j = i * 8 + qc * 2 + c;
      s[i][c] = j <= i0 ? s[i][c] * power[i0 - j] : 0.f;
      s[i][2 + c] = j <= i1 ? s[i][2 + c] * power[i1 - j] : 0.f;
    }
  }
#pragma unroll
  for (int kk = 0; kk < DC / 16; kk++) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int d2 = 0; d2 < DVB / 16; d2++) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
      mma_bf16(o[2 * d2], a, b[0], b[1]);
      mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
    }
  }
#pragma unroll
  for (int half = 0; half < 2; half++) {
    const int i = half ? i1 : i0;
    if (i >= n) continue;
    float* dst = out + (size_t)(t0 + i) * heads * vdim + (size_t)h * vdim + col0;
#pragma unroll
    for (int nt = 0; nt < DVB / 8; nt++) {
      const int col = nt * 8 + qc * 2;
      if (col0 + col < vdim) *(float2*)(dst + col) = make_float2(o[nt][half * 2], o[nt][half * 2 + 1]);
    }
  }
}

template <int DIM>
int launch_chunks_at_once(const void* rows, int row_stride, const int* q_start, const int* state_slots, float* state,
                          int num_slots, const float* decay, float* out, float* sums, int max_chunks, int requests, int heads,
                          int vdim, int* status, cudaStream_t stream) {
  const int smem_sums = (3 * DC * (DIM + 8) + DC * (DVB + 8)) * 2;
  const int smem_out = (2 * DC * (DIM + 8) + DC * (DVB + 8) + 2 * DIM * (DVB + 8)) * 2;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(decay_chunk_sums_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_sums);
    cudaFuncSetAttribute(decay_chunk_outputs_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_out);
    configured = true;
  }
  const int blocks = (vdim + DVB - 1) / DVB, plane = DIM * vdim;
  sprout_launch(decay_chunk_sums_kernel<DIM>, dim3(max_chunks, heads, blocks), dim3(DC_THREADS), smem_sums, stream,
                (const __nv_bfloat16*)rows, row_stride, q_start, requests, decay, sums, heads, vdim);
  if (int code = sprout_check_launch("decay_chunk_sums")) return code;
  sprout_launch(decay_chunk_scan_kernel, dim3(requests, heads, (plane + 255) / 256), dim3(256), 0, stream, q_start, state_slots,
                state, num_slots, decay, sums, heads, plane, status);
  if (int code = sprout_check_launch("decay_chunk_scan")) return code;
  sprout_launch(decay_chunk_outputs_kernel<DIM>, dim3(max_chunks, heads, blocks), dim3(DC_THREADS), smem_out, stream,
                (const __nv_bfloat16*)rows, row_stride, q_start, requests, decay, (const float*)sums, out, heads, vdim);
  return sprout_check_launch("decay_chunk_outputs");
}

template <int DIM>
int launch_chunks(const void* rows, int row_stride, const int* q_start, const int* state_slots, float* state, int num_slots,
                  const float* decay, float* out, int requests, int heads, int vdim, int* status, cudaStream_t stream) {
  const int smem = (6 * DC * (DIM + 8) + 2 * DC * (DVB + 8) + 2 * DIM * (DVB + 8)) * 2;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(decay_chunks_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured = true;
  }
  sprout_launch(decay_chunks_kernel<DIM>, dim3(requests, heads, (vdim + DVB - 1) / DVB), dim3(DC_THREADS), smem, stream,
                (const __nv_bfloat16*)rows, row_stride, q_start, state_slots, state, num_slots, decay, out, heads, vdim, status);
  return sprout_check_launch("decay_chunks");
}

}  // namespace

// The chunked kernel copies 16-byte pieces of the rows: key vectors of 64 or 128, value rows and row strides in multiples of 8.
SPROUT_API int sprout_decay_chunks_supported(int dim, int vdim, int row_stride) {
  return (dim == 64 || dim == 128) && vdim % 8 == 0 && row_stride % 8 == 0;
}

// The same as decay_scan for bfloat16 rows, 64 tokens at a time on tensor cores.  With `act` the first
// heads * (2 dim + vdim) elements of every row are replaced by their activation first (in place).
// With `sums` (float32 scratch [max_chunks, heads, dim, vdim], max_chunks >= the sum over requests of ceil(tokens / 64)) all chunks run
// at once in three launches; without it a CTA walks its request's chunks in order with the state in registers.
SPROUT_API int sprout_decay_chunks(void* rows, int row_stride, const int* q_start, const int* state_slots, float* state,
                                   int num_slots, const float* decay, float* out, float* sums, int max_chunks, int tokens,
                                   int requests, int heads, int dim, int vdim, int act, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(rows && q_start && state_slots && state && decay && out && status, "decay_chunks: null pointer");
  SPROUT_REQUIRE(tokens > 0 && requests > 0 && heads > 0 && vdim > 0 && num_slots > 0 && heads <= 65535, "decay_chunks: bad sizes");
  SPROUT_REQUIRE(row_stride >= heads * (2 * dim + vdim), "decay_chunks: rows too short");
  SPROUT_REQUIRE(sprout_decay_chunks_supported(dim, vdim, row_stride) && ((uintptr_t)rows & 15) == 0 && ((uintptr_t)out & 7) == 0,
                 "decay_chunks: key vectors of 64 or 128 elements, rows in 16-byte pieces (dim %d, vdim %d, stride %d)", dim, vdim, row_stride);
  if (act) {
    const int width8 = heads * (2 * dim + vdim) / 8;                 // a multiple of 8: dim is, vdim is
    const long long count8 = (long long)tokens * width8;
    const int grid = (int)((count8 + 255) / 256 < 148 * 16 ? (count8 + 255) / 256 : 148 * 16);
    sprout_launch(silu_rows_kernel, dim3(grid), dim3(256), 0, stream, (__nv_bfloat16*)rows, row_stride, width8, count8);
    if (int code = sprout_check_launch("silu_rows")) return code;
  }
  if (sums) {
    SPROUT_REQUIRE(max_chunks > 0 && ((uintptr_t)sums & 7) == 0 && vdim % 2 == 0, "decay_chunks: the sums' scratch is too small or misaligned");
    if (dim == 64)
      return launch_chunks_at_once<64>(rows, row_stride, q_start, state_slots, state, num_slots, decay, out, sums, max_chunks, requests,
                                       heads, vdim, status, stream);
    return launch_chunks_at_once<128>(rows, row_stride, q_start, state_slots, state, num_slots, decay, out, sums, max_chunks, requests,
                                      heads, vdim, status, stream);
  }
  if (dim == 64)
    return launch_chunks<64>(rows, row_stride, q_start, state_slots, state, num_slots, decay, out, requests, heads, vdim, status, stream);
  return launch_chunks<128>(rows, row_stride, q_start, state_slots, state, num_slots, decay, out, requests, heads, vdim, status, stream);
}

// rows [tokens, row_stride] (dtype), out float32 [tokens, heads * vdim], state float32 [slots, heads, dim, vdim].
SPROUT_API int sprout_decay_scan(const void* rows, int row_stride, int dtype, const int* q_start, const int* state_slots,
                                 float* state, int num_slots, const float* decay, float* out, int requests, int heads,
                                 int dim, int vdim, int act, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(rows && q_start && state_slots && state && decay && out && status, "decay_scan: null pointer");
  SPROUT_REQUIRE(requests > 0 && heads > 0 && dim > 0 && vdim > 0 && num_slots > 0, "decay_scan: sizes must be positive");
  SPROUT_REQUIRE(row_stride >= heads * (2 * dim + vdim), "decay_scan: rows too short");
  SPROUT_REQUIRE(heads <= 65535, "decay_scan: too many heads");
  int cols = 32;
  while (cols < vdim && cols < 128) cols *= 2;
  while ((size_t)(dim * cols + 2 * dim) * sizeof(float) > 200 * 1024 && cols > 32) cols /= 2;
  const size_t smem = (size_t)(dim * cols + 2 * dim) * sizeof(float);
  SPROUT_REQUIRE(smem <= 200 * 1024, "decay_scan: key vectors too long (%d)", dim);
  dim3 grid(requests, heads, (vdim + cols - 1) / cols);
  if (dtype == SPROUT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sprout_launch(decay_scan_kernel<float>, grid, dim3(cols), smem, stream, (const float*)rows, row_stride, q_start,
                  state_slots, state, num_slots, decay, out, heads, dim, vdim, act, status);
  } else if (dtype == SPROUT_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(decay_scan_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    sprout_launch(decay_scan_kernel<__nv_bfloat16>, grid, dim3(cols), smem, stream, (const __nv_bfloat16*)rows, row_stride,
                  q_start, state_slots, state, num_slots, decay, out, heads, dim, vdim, act, status);
  } else {
    return sprout_fail("decay_scan: unknown dtype %d", dtype);
  }
  return sprout_check_launch("decay_scan");
}
