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
//                 A CTA owns (request, head, 32 value columns) and keeps its part of S in accumulator registers
//                 (float32) from chunk to chunk.  What enters the recurrence stays 32-bit in effect: the decayed keys
//                 and the state read by the queries go to the tensor cores as two bfloat16 terms each (value = high +
//                 low), so their rounding is 2^-17, not 2^-9; the decay powers are float32.
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
constexpr int DC = 64, DVB = 32, DC_THREADS = 128;     // tokens per chunk, value columns per CTA

template <int DIM>
__global__ void __launch_bounds__(DC_THREADS)
decay_chunks_kernel(const __nv_bfloat16* __restrict__ rows, int row_stride, const int* __restrict__ q_start,
                    const int* __restrict__ state_slots, float* __restrict__ state, int num_slots,
                    const float* __restrict__ decay, float* __restrict__ out, int heads, int vdim, int act, int* status) {
  constexpr int QS = DIM + 8, VS = DVB + 8, MT = DIM / 64;        // a warp owns DIM / 4 rows of the state: MT tiles of 16
  extern __shared__ __align__(16) unsigned char dc_smem[];
  __nv_bfloat16* sQ = (__nv_bfloat16*)dc_smem;                    // DC x QS
  __nv_bfloat16* sK = sQ + DC * QS;
  __nv_bfloat16* sKh = sK + DC * QS;                              // decayed keys, high and low terms
  __nv_bfloat16* sKl = sKh + DC * QS;
  __nv_bfloat16* sV = sKl + DC * QS;                              // DC x VS
  __nv_bfloat16* sSh = sV + DC * VS;                              // DIM x VS: the state, high and low terms
  __nv_bfloat16* sSl = sSh + DIM * VS;
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * DVB;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, gr = lane >> 2, qc = lane & 3;
  const int slot = state_slots[r];
  if (slot < 0 || slot >= num_slots) {
    if (tid == 0) atomicOr(status, SPROUT_STATUS_BAD_PAGE);
    return;
  }
  float* mine = state + (((size_t)slot * heads + h) * DIM) * vdim;
  const float lam = decay[h], log_lam = log2f(lam);
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
  for (int t0 = first; t0 < last; t0 += DC) {
    const int n = min(DC, last - t0);
    __syncthreads();                                   // the chunk before is done with shared memory
    // q, k (activated, as bfloat16 holds them), the decayed keys in two terms, v
    for (int idx = tid; idx < DC * DIM; idx += DC_THREADS) {
      const int j = idx / DIM, d = idx % DIM;
      float q = 0.f, k = 0.f;
      if (j < n) {
        const __nv_bfloat16* row = rows + (size_t)(t0 + j) * row_stride + (size_t)h * DIM + d;
        q = activate(row[0], act);
        k = activate(row[(size_t)heads * DIM], act);
      }
      sQ[j * QS + d] = __float2bfloat16_rn(q);
      sK[j * QS + d] = __float2bfloat16_rn(k);
      const float kd = k * exp2f((float)(n - 1 - j) * log_lam);
      const __nv_bfloat16 hi = __float2bfloat16_rn(kd);
      sKh[j * QS + d] = hi;
      sKl[j * QS + d] = __float2bfloat16_rn(kd - __bfloat162float(hi));
    }
    for (int idx = tid; idx < DC * DVB; idx += DC_THREADS) {
      const int j = idx / DVB, c = idx % DVB;
      float v = 0.f;
      if (j < n && col0 + c < vdim) v = activate(rows[(size_t)(t0 + j) * row_stride + (size_t)2 * heads * DIM + (size_t)h * vdim + col0 + c], act);
      sV[j * VS + c] = __float2bfloat16_rn(v);
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
      ldmatrix_x4(a, sQ + (warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * QS + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int n2 = 0; n2 < DC / 16; n2++) {
        uint32_t b[4];
        ldmatrix_x4(b, sK + (n2 * 16 + (lane & 7) + (lane >> 4) * 8) * QS + kk * 16 + ((lane >> 3) & 1) * 8);
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
    const float carry0 = exp2f((float)(i0 + 1) * log_lam), carry1 = exp2f((float)(i1 + 1) * log_lam);
#pragma unroll
    for (int i = 0; i < DVB / 8; i++) { o[i][0] *= carry0; o[i][1] *= carry0; o[i][2] *= carry1; o[i][3] *= carry1; }
#pragma unroll
    for (int i = 0; i < DC / 8; i++) {
#pragma unroll
      for (int c = 0; c < 2; c++) {
        const int j = i * 8 + qc * 2 + c;
        s[i][c] = j <= i0 ? s[i][c] * exp2f((float)(i0 - j) * log_lam) : 0.f;
        s[i][2 + c] = j <= i1 ? s[i][2 + c] * exp2f((float)(i1 - j) * log_lam) : 0.f;
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
        if (col0 + col < vdim) dst[col] = o[nt][half * 2];
        if (col0 + col + 1 < vdim) dst[col + 1] = o[nt][half * 2 + 1];
      }
    }

    // the state after the chunk: decay^n S + (decayed keys)^T V, the keys' two terms one after the other
    const float shrink = exp2f((float)n * log_lam);
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
          ldmatrix_x4_trans(b, sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * VS + d2 * 16 + (lane >> 4) * 8);
          mma_bf16(S[mt][2 * d2], ah, b[0], b[1]);
          mma_bf16(S[mt][2 * d2 + 1], ah, b[2], b[3]);
          mma_bf16(S[mt][2 * d2], al, b[0], b[1]);
          mma_bf16(S[mt][2 * d2 + 1], al, b[2], b[3]);
        }
      }
    }
  }
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

template <int DIM>
int launch_chunks(const void* rows, int row_stride, const int* q_start, const int* state_slots, float* state, int num_slots,
                  const float* decay, float* out, int requests, int heads, int vdim, int act, int* status, cudaStream_t stream) {
  const int smem = (4 * DC * (DIM + 8) + DC * (DVB + 8) + 2 * DIM * (DVB + 8)) * 2;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(decay_chunks_kernel<DIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    configured = true;
  }
  sprout_launch(decay_chunks_kernel<DIM>, dim3(requests, heads, (vdim + DVB - 1) / DVB), dim3(DC_THREADS), smem, stream,
                (const __nv_bfloat16*)rows, row_stride, q_start, state_slots, state, num_slots, decay, out, heads, vdim, act, status);
  return sprout_check_launch("decay_chunks");
}

}  // namespace

SPROUT_API int sprout_decay_chunks_supported(int dim) { return dim == 64 || dim == 128; }

// The same as decay_scan for bfloat16 rows, 64 tokens at a time on tensor cores.
SPROUT_API int sprout_decay_chunks(const void* rows, int row_stride, const int* q_start, const int* state_slots, float* state,
                                   int num_slots, const float* decay, float* out, int requests, int heads, int dim, int vdim,
                                   int act, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(rows && q_start && state_slots && state && decay && out && status, "decay_chunks: null pointer");
  SPROUT_REQUIRE(requests > 0 && heads > 0 && vdim > 0 && num_slots > 0 && heads <= 65535, "decay_chunks: bad sizes");
  SPROUT_REQUIRE(row_stride >= heads * (2 * dim + vdim), "decay_chunks: rows too short");
  if (dim == 64)
    return launch_chunks<64>(rows, row_stride, q_start, state_slots, state, num_slots, decay, out, requests, heads, vdim, act, status, stream);
  if (dim == 128)
    return launch_chunks<128>(rows, row_stride, q_start, state_slots, state, num_slots, decay, out, requests, heads, vdim, act, status, stream);
  return sprout_fail("decay_chunks: key vectors of 64 or 128 elements (got %d)", dim);
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
