// Linear attention with a per-head decay and a state per request ("lightning attention"):
//   S_t = decay_h * S_(t-1) + k_t v_t^T,   o_t = S_t^T q_t        (S: [dim, vdim] per head, float32)
// with q, k, v = act(projection) (act = silu, or none).  The state of a request lives in a slot of a
// buffer [slots, heads, dim, vdim]; a step reads it, runs the request's tokens of this step and writes it
// back, so a prompt may be cut anywhere.
//
//  * decay_scan:  one block per (request, head, block of value columns), token by token in float32: thread j
//                 owns column j of the state; the order of operations per element is the tokens' order, so the
//                 result does not depend on the cutting or on the batch.
// A token's row holds [q: heads * dim | k: heads * dim | v: heads * vdim | ...] as the projection left it.
#include "common.cuh"

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

}  // namespace

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
