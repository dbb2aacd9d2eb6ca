// Latent attention on tensor cores (mma.sync.m16n8k16, bfloat16 operands, float32 accumulation and softmax).
//
// The cache holds one row per token, `width` = rank + rot wide, shared by all heads; a query row
// (token, head) is as wide; its score with a key row is their dot product times `scale`; the value of a
// key row is its first `rank` elements.  Rows of a request's tokens are tiled 16 to a warp; all rows of
// a tile read the same staged key rows (cp.async, double-buffered stages of KEYS rows), once for the
// scores (ldmatrix) and once, transposed, as values.  A CTA accumulates DVC value columns; a latent
// wider than a CTA's blocks is divided among CTAs (blockIdx.y), each of which computes the scores again.
//
//  * whole rows (prefill and mixed batches): a CTA of 8 warps owns 128 rows of one request, or 64 rows
//    with each half of the warps taking one of two blocks of DVC value columns (both halves compute the
//    scores; the staged keys and the query rows are shared), and walks the keys up to its last row's
//    position; a head's sink starts the running maximum and sum.
//  * split keys (one token per request): a CTA owns the 16 heads of a request's token and one range of
//    its keys; 4 warps per block of value columns take a quarter of every stage each and are merged
//    through shared memory; the ranges' partial sums go through float32 scratch to a merge kernel,
//    which also adds the sink.
#include "attention_bf16.cuh"
#include "tcgen05.cuh"

using namespace sprout_attn;

namespace {

constexpr int WARPS = 8;          // of a whole-rows CTA

struct LatentParams {
  const __nv_bfloat16* q;         // [tokens, heads * width]
  const __nv_bfloat16* cache;     // [pages, 1, page_tokens, width]
  const int* block_table; int table_stride;
  const int* q_start;             // [requests + 1]
  const int* positions;           // [tokens]
  const int* context_lens;        // [requests] (split keys)
  const float* sink;              // [heads] or null
  __nv_bfloat16* out;             // [tokens, heads * rank]
  float* part_o;                  // [requests, splits, heads, rank]   (split keys)
  float* part_ml;                 // [requests, splits, heads, 2]
  int requests, heads, width, rank, page_tokens, num_pages, split_keys, splits;
  float scale;
  int* status;
};

// One warp: scores of its 16 rows against NT * 8 staged keys over the k-steps [kk0, kk1) of the rows' width.
template <int NT>
__device__ __forceinline__ void scores_block(const __nv_bfloat16* sQ, const __nv_bfloat16* tK, int stride, int kk0, int kk1,
                                             float (&s)[NT][4], int lane) {
#pragma unroll
  for (int i = 0; i < NT; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
  const __nv_bfloat16* a_ptr = sQ + ((lane & 7) + ((lane >> 3) & 1) * 8) * stride + (lane >> 4) * 8;
  const __nv_bfloat16* b_ptr = tK + ((lane & 7) + (lane >> 4) * 8) * stride + ((lane >> 3) & 1) * 8;
  if (NT == 2) {
    // one pair of tiles: four k-steps at a time go to accumulators of their own (four chains instead of one)
    float c[3][2][4];
#pragma unroll
    for (int i = 0; i < 3; i++)
#pragma unroll
      for (int j = 0; j < 4; j++) c[i][0][j] = c[i][1][j] = 0.f;
    int kk = kk0;
    for (; kk + 3 < kk1; kk += 4) {
      uint32_t a[4][4], b[4][4];
#pragma unroll
      for (int u = 0; u < 4; u++) { ldmatrix_x4(a[u], a_ptr + (kk + u) * 16); ldmatrix_x4(b[u], b_ptr + (kk + u) * 16); }
      mma_bf16(s[0], a[0], b[0][0], b[0][1]);
      mma_bf16(s[1], a[0], b[0][2], b[0][3]);
#pragma unroll
      for (int u = 1; u < 4; u++) {
        mma_bf16(c[u - 1][0], a[u], b[u][0], b[u][1]);
        mma_bf16(c[u - 1][1], a[u], b[u][2], b[u][3]);
      }
    }
    for (; kk < kk1; kk++) {
      uint32_t a[4], b[4];
      ldmatrix_x4(a, a_ptr + kk * 16);
      ldmatrix_x4(b, b_ptr + kk * 16);
      mma_bf16(s[0], a, b[0], b[1]);
      mma_bf16(s[1], a, b[2], b[3]);
    }
#pragma unroll
    for (int j = 0; j < 4; j++) {
      s[0][j] += (c[0][0][j] + c[1][0][j]) + c[2][0][j];
      s[1][j] += (c[0][1][j] + c[1][1][j]) + c[2][1][j];
    }
  } else {
#pragma unroll 2
    for (int kk = kk0; kk < kk1; kk++) {
      uint32_t a[4];
      ldmatrix_x4(a, a_ptr + kk * 16);
#pragma unroll
      for (int n2 = 0; n2 < NT / 2; n2++) {
        uint32_t b[4];
        ldmatrix_x4(b, b_ptr + n2 * 16 * stride + kk * 16);
        mma_bf16(s[2 * n2], a, b[0], b[1]);
        mma_bf16(s[2 * n2 + 1], a, b[2], b[3]);
      }
    }
  }
}

// The same warp, from its scores on: mask, online softmax, O += P V over the warp's value columns.
template <int DVC, int NT>
__device__ __forceinline__ void softmax_values_block(float (&s)[NT][4], const __nv_bfloat16* tK, int stride, int col0, int col_end,
                                                     int key0, int limit0, int limit1, bool mask, float scale_log2, float& m0,
                                                     float& m1, float& l0, float& l1, float (&o)[DVC / 8][4], int lane) {
  const int qc = lane & 3;
  if (mask) {
#pragma unroll
    for (int i = 0; i < NT; i++) {
      const int key = key0 + i * 8 + qc * 2;
      if (key > limit0) s[i][0] = -INFINITY;
      if (key + 1 > limit0) s[i][1] = -INFINITY;
      if (key > limit1) s[i][2] = -INFINITY;
      if (key + 1 > limit1) s[i][3] = -INFINITY;
    }
  }
  float t0 = -INFINITY, t1 = -INFINITY;
#pragma unroll
  for (int i = 0; i < NT; i++) {
    t0 = fmaxf(t0, fmaxf(s[i][0], s[i][1]));
    t1 = fmaxf(t1, fmaxf(s[i][2], s[i][3]));
  }
  t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
  t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
  t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
  t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
  const float n0 = fmaxf(m0, t0), n1 = fmaxf(m1, t1);          // running maxima of the unscaled scores
  const float base0 = n0 == -INFINITY ? 0.f : n0 * scale_log2, base1 = n1 == -INFINITY ? 0.f : n1 * scale_log2;
  const float alpha0 = m0 == -INFINITY ? 0.f : exp2f(m0 * scale_log2 - base0);
  const float alpha1 = m1 == -INFINITY ? 0.f : exp2f(m1 * scale_log2 - base1);
  m0 = n0; m1 = n1;
  l0 *= alpha0; l1 *= alpha1;
  if (!__all_sync(0xffffffffu, alpha0 == 1.f && alpha1 == 1.f)) {       // most blocks move no row's maximum
#pragma unroll
    for (int i = 0; i < DVC / 8; i++) { o[i][0] *= alpha0; o[i][1] *= alpha0; o[i][2] *= alpha1; o[i][3] *= alpha1; }
  }
#pragma unroll
  for (int i = 0; i < NT; i++) {
    s[i][0] = exp2f(fmaf(s[i][0], scale_log2, -base0)); s[i][1] = exp2f(fmaf(s[i][1], scale_log2, -base0));
    s[i][2] = exp2f(fmaf(s[i][2], scale_log2, -base1)); s[i][3] = exp2f(fmaf(s[i][3], scale_log2, -base1));
    l0 += s[i][0] + s[i][1];
    l1 += s[i][2] + s[i][3];
  }
  const __nv_bfloat16* v_ptr = tK + ((lane & 7) + ((lane >> 3) & 1) * 8) * stride + col0 + (lane >> 4) * 8;
#pragma unroll
  for (int kk = 0; kk < NT / 2; kk++) {
    uint32_t a[4];
    a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
    a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
    a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
    a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
    for (int d2 = 0; d2 < DVC / 16; d2++) {
      if (col0 + d2 * 16 < col_end) {
        uint32_t b[4];
        ldmatrix_x4_trans(b, v_ptr + kk * 16 * stride + d2 * 16);
        mma_bf16(o[2 * d2], a, b[0], b[1]);
        mma_bf16(o[2 * d2 + 1], a, b[2], b[3]);
      }
    }
  }
}

template <int DVC, int NT>
__device__ __forceinline__ void attend_block(const __nv_bfloat16* sQ, const __nv_bfloat16* tK, int stride, int width,
                                             int col0, int col_end, int key0, int limit0, int limit1, bool mask,
                                             float scale_log2, float& m0, float& m1, float& l0, float& l1,
                                             float (&o)[DVC / 8][4], int lane) {
  float s[NT][4];
  scores_block<NT>(sQ, tK, stride, 0, width / 16, s, lane);
  softmax_values_block<DVC, NT>(s, tK, stride, col0, col_end, key0, limit0, limit1, mask, scale_log2, m0, m1, l0, l1, o, lane);
}

// One stage of key rows: each of the first KEYS threads finds its row's place in the pool and starts one bulk copy
// of the whole row into shared memory (a row beyond the range is cleared instead); every one of them arrives on the
// stage's mbarrier (initialised with a count of KEYS), a copying thread together with its row's bytes.
__device__ __forceinline__ void bulk_row(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// The page of a thread's key row in a stage (read one stage ahead of its use, so that the load's latency is not on the
// stage's path): -2 for a key beyond the range, else the block table's entry.
template <int KEYS>
__device__ __forceinline__ int page_ahead(const LatentParams& p, const int* table, int first_key, int last_key, int tid) {
  const int key = first_key + tid;
  return (tid < KEYS && key <= last_key) ? table[key / p.page_tokens] : -2;
}
template <int KEYS>
__device__ __forceinline__ void issue_stage(const LatentParams& p, int page, int first_key, __nv_bfloat16* dst, int stride,
                                            uint64_t* bar, int tid) {
  if (tid < KEYS) {
    const int key = first_key + tid;
    long long off = -1;
    if (page != -2) {
      if (page < 0 || page >= p.num_pages) atomicOr(p.status, SPROUT_STATUS_BAD_PAGE);
      else off = ((long long)page * p.page_tokens + key % p.page_tokens) * p.width;
    }
    __nv_bfloat16* d = dst + tid * stride;
    if (off >= 0) {
      mbar_expect_tx(bar, (uint32_t)p.width * 2);
      bulk_row(d, p.cache + off, (uint32_t)p.width * 2, bar);
    } else {
      for (int c = 0; c < p.width / 8; c++) ((uint4*)d)[c] = make_uint4(0, 0, 0, 0);
      mbar_arrive(bar);
    }
  }
}
// All threads wait for a stage.  A wait that runs out flags the status word and the CTA's `failed` flag, which every
// thread reads after the next barrier: the CTA then stops walking keys, all its threads at the same stage.
__device__ __forceinline__ void stage_landed(uint64_t* bar, uint32_t parity, int* status, volatile int* failed) {
  if (mbar_wait(bar, parity)) return;
  *failed = 1;
  atomicOr(status, SPROUT_STATUS_WAIT_TIMEOUT);
}
// rows [0, rows) of 16-byte pieces: thread tid takes pieces tid, tid + threads, ... (row and piece advance without a division)
template <typename F>
__device__ __forceinline__ void for_pieces(int rows, int pieces, int tid, int threads, F f) {
  int row = tid / pieces, c = tid % pieces;
  const int drow = threads / pieces, dc = threads % pieces;
  while (row < rows) {
    f(row, c);
    row += drow; c += dc;
    if (c >= pieces) { c -= pieces; row++; }
  }
}
// ------------------------------------------------------------------------------ whole rows
template <int DVC, int KEYS, int CHUNKS>
__global__ void __launch_bounds__(WARPS * 32)
latent_attention_rows_kernel(const LatentParams p) {
  constexpr int THREADS = WARPS * 32, GROUPS = WARPS / CHUNKS, ROWS = GROUPS * 16;
  extern __shared__ __align__(16) uint8_t lsm[];
  const int stride = p.width + 8;
  __nv_bfloat16* sQ = (__nv_bfloat16*)lsm;            // [ROWS][stride]
  __nv_bfloat16* sK = sQ + ROWS * stride;             // [2][KEYS][stride]
  __shared__ int s_limit[ROWS];
  __shared__ int s_token[ROWS];
  __shared__ int s_head[ROWS];
  __shared__ __align__(8) uint64_t s_bar[2];
  __shared__ int s_failed;
  // with two blocks of value columns: a warp's partial scores, for the warp that has the same rows and the other block
  __shared__ __align__(16) float s_part[CHUNKS == 2 ? WARPS : 1][CHUNKS == 2 ? KEYS * 16 : 4];

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    s_failed = 0;
    mbar_init(&s_bar[0], KEYS);
    mbar_init(&s_bar[1], KEYS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();
  const int group = warp % GROUPS;                    // which 16 rows
  const int col0 = (blockIdx.y * CHUNKS + warp / GROUPS) * DVC, col_end = min(p.rank, col0 + DVC);

  int r = 0, tile = blockIdx.x;
  for (; r < p.requests; r++) {
    const int tiles = ((p.q_start[r + 1] - p.q_start[r]) * p.heads + ROWS - 1) / ROWS;
    if (tile < tiles) {
      tile = (tile & 1) ? tiles - 1 - (tile >> 1) : (tile >> 1);      // long and short tiles alternate in launch order
      break;
    }
    tile -= tiles;
  }
  if (r >= p.requests) return;
  const int q0 = p.q_start[r], rows_total = (p.q_start[r + 1] - q0) * p.heads;
  const int row_base = tile * ROWS;
  const int* table = p.block_table + (size_t)r * p.table_stride;
  if (tid < ROWS) {
    const int gi = row_base + tid;
    if (gi < rows_total) {
      const int tok = q0 + gi / p.heads;
      s_token[tid] = tok; s_head[tid] = gi % p.heads; s_limit[tid] = p.positions[tok];
    } else {
      s_token[tid] = -1; s_head[tid] = 0; s_limit[tid] = -1;
    }
  }
  __syncthreads();
  const int last_row = min(rows_total, row_base + ROWS) - 1 - row_base;
  const int max_limit = s_limit[last_row];
  const int stages = max_limit / KEYS + 1;
  for_pieces(ROWS, p.width / 8, tid, THREADS, [&](int row, int c) {
    __nv_bfloat16* dst = sQ + row * stride + c * 8;
    if (s_token[row] >= 0) cp_async16(dst, p.q + ((size_t)s_token[row] * p.heads + s_head[row]) * p.width + c * 8);
    else *(uint4*)dst = make_uint4(0, 0, 0, 0);
  });
  cp_async_commit();
  issue_stage<KEYS>(p, page_ahead<KEYS>(p, table, 0, max_limit, tid), 0, sK, stride, &s_bar[0], tid);
  int page_next = page_ahead<KEYS>(p, table, KEYS, max_limit, tid);       // of the stage after: read now, used at the loop's next turn
  cp_async_wait<0>();                                 // this thread's pieces of the query rows; the loop's first barrier publishes them

  const int gr = lane >> 2, qc = lane & 3;
  const int my_row0 = group * 16 + gr, my_row1 = my_row0 + 8;
  const int limit0 = s_limit[my_row0], limit1 = s_limit[my_row1];
  const float scale_log2 = p.scale * 1.4426950408889634f;
  // a sink starts the running maximum (in units of the unscaled score) and counts once in the sum
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  if (p.sink) {
    m0 = p.sink[s_head[my_row0]] / p.scale; m1 = p.sink[s_head[my_row1]] / p.scale;
    if (qc == 0) { l0 = 1.f; l1 = 1.f; }
  }
  float o[DVC / 8][4];
#pragma unroll
  for (int i = 0; i < DVC / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int warp_min_limit = s_limit[min(group * 16, last_row)];
  const int warp_limit = s_limit[min(group * 16 + 15, last_row)];
  const bool active = group * 16 <= last_row && col0 < p.rank;
  const bool paired = CHUNKS == 2 && (blockIdx.y * CHUNKS + 1) * DVC < p.rank;      // both blocks of value columns exist

  for (int t = 0; t < stages; t++) {
    const int buf = t & 1;
    __syncthreads();                                  // every warp is done with the other buffer; cleared rows are visible
    if (s_failed) break;
    if (t + 1 < stages) {
      issue_stage<KEYS>(p, page_next, (t + 1) * KEYS, sK + (buf ^ 1) * KEYS * stride, stride, &s_bar[buf ^ 1], tid);
      page_next = page_ahead<KEYS>(p, table, (t + 2) * KEYS, max_limit, tid);
    }
    stage_landed(&s_bar[buf], (t >> 1) & 1, p.status, &s_failed);
    const int key0 = t * KEYS;
    if (active && key0 <= warp_limit) {
      constexpr int NT = KEYS / 8;
      const __nv_bfloat16* tK = sK + buf * KEYS * stride;
      float sc[NT][4];
      if (CHUNKS == 2 && paired) {
        // the two warps with the same rows take half of the rows' width each and add their partial scores through
        // shared memory: the scores are computed once per CTA, not once per block of value columns
        const int steps = p.width / 16, half = (steps + 1) / 2;
        scores_block<NT>(sQ + group * 16 * stride, tK, stride, warp >= GROUPS ? half : 0, warp >= GROUPS ? steps : half, sc, lane);
        float4* mine = (float4*)s_part[CHUNKS == 2 ? warp : 0];
#pragma unroll
        for (int i = 0; i < NT; i++) mine[i * 32 + lane] = make_float4(sc[i][0], sc[i][1], sc[i][2], sc[i][3]);
        asm volatile("bar.sync %0, 64;" ::"r"(1 + group) : "memory");
        const float4* other = (const float4*)s_part[CHUNKS == 2 ? (warp + GROUPS) % WARPS : 0];
#pragma unroll
        for (int i = 0; i < NT; i++) {
          const float4 u = other[i * 32 + lane];
          sc[i][0] += u.x; sc[i][1] += u.y; sc[i][2] += u.z; sc[i][3] += u.w;
        }
      } else {
        scores_block<NT>(sQ + group * 16 * stride, tK, stride, 0, p.width / 16, sc, lane);
      }
      softmax_values_block<DVC, NT>(sc, tK, stride, col0, col_end, key0, limit0, limit1, key0 + KEYS - 1 > warp_min_limit,
                                    scale_log2, m0, m1, l0, l1, o, lane);
    }
  }
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  if (!active) return;
#pragma unroll
  for (int half = 0; half < 2; half++) {
    const int row = half ? my_row1 : my_row0;
    if (s_token[row] < 0) continue;
    __nv_bfloat16* dst = p.out + ((size_t)s_token[row] * p.heads + s_head[row]) * p.rank + col0 + qc * 2;
    const float inv = 1.0f / (half ? l1 : l0);
#pragma unroll
    for (int i = 0; i < DVC / 8; i++)
      if (col0 + i * 8 < col_end)
        *(__nv_bfloat162*)(dst + i * 8) = __floats2bfloat162_rn(o[i][half * 2] * inv, o[i][half * 2 + 1] * inv);
  }
}

// ------------------------------------------------------------------------------ split keys (one token per request)
// PARTS warps per block of value columns take 16 keys of a stage each (KEYS = 16 PARTS); NSTAGES buffers, of which
// NSTAGES - 1 are on their way while one is worked on.
template <int DVC, int CHUNKS, int PARTS, int NSTAGES>
__global__ void __launch_bounds__(CHUNKS * PARTS * 32, 4 / CHUNKS)        // 128 registers a thread: 16 warps on an SM
latent_attention_split_kernel(const LatentParams p) {
  constexpr int KEYS = 16 * PARTS, THREADS = CHUNKS * PARTS * 32;
  extern __shared__ __align__(16) uint8_t lsm[];
  const int stride = p.width + 8;
  __nv_bfloat16* sQ = (__nv_bfloat16*)lsm;            // [16][stride]
  __nv_bfloat16* sK = sQ + 16 * stride;               // [NSTAGES][KEYS][stride]; after the loop: the warps' partial sums
  __shared__ __align__(8) uint64_t s_bar[NSTAGES];
  __shared__ int s_failed;
  __shared__ float s_ml[PARTS][16][2];
  __shared__ __align__(16) float s_part[CHUNKS * PARTS][256];   // a warp's partial scores, for the warp that shares its keys

  pdl_launch_dependents();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) {
    s_failed = 0;
    for (int i = 0; i < NSTAGES; i++) mbar_init(&s_bar[i], KEYS);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_wait();
  const int quarter = warp % PARTS, chunk = warp / PARTS;    // which 16 keys of a stage, which block of value columns
  const int groups = (p.heads + 15) / 16;
  const int r = blockIdx.x / groups, head0 = (blockIdx.x % groups) * 16;
  const int cta_col0 = blockIdx.y * CHUNKS * DVC, cta_col_end = min(p.rank, cta_col0 + CHUNKS * DVC);
  const int col0 = cta_col0 + chunk * DVC, col_end = min(p.rank, col0 + DVC);
  const int split = blockIdx.z;
  const int limit = p.context_lens[r] - 1;            // the token's own position: the last key it sees
  // the last range runs to the token's position, however the ranges were planned
  const int first = split * p.split_keys, last = split == p.splits - 1 ? limit : min(limit, first + p.split_keys - 1);
  const int stages = last >= first ? (last - first) / KEYS + 1 : 0;
  const int* table = p.block_table + (size_t)r * p.table_stride;
  const int token = p.q_start[r];
  for_pieces(16, p.width / 8, tid, THREADS, [&](int row, int c) {
    __nv_bfloat16* dst = sQ + row * stride + c * 8;
    if (head0 + row < p.heads) cp_async16(dst, p.q + ((size_t)token * p.heads + head0 + row) * p.width + c * 8);
    else *(uint4*)dst = make_uint4(0, 0, 0, 0);
  });
  cp_async_commit();
  __syncthreads();                                    // the mbarriers are initialised
  for (int t = 0; t < NSTAGES - 1 && t < stages; t++)
    issue_stage<KEYS>(p, page_ahead<KEYS>(p, table, first + t * KEYS, last, tid), first + t * KEYS, sK + t * KEYS * stride, stride,
                      &s_bar[t], tid);
  int page_next = page_ahead<KEYS>(p, table, first + (NSTAGES - 1) * KEYS, last, tid);   // read now, used at the loop's next turn
  cp_async_wait<0>();

  const int gr = lane >> 2, qc = lane & 3;
  const float scale_log2 = p.scale * 1.4426950408889634f;
  const int steps = p.width / 16;
  const bool shared_scores = CHUNKS > 1 && cta_col0 + (CHUNKS - 1) * DVC < p.rank;      // all the CTA's blocks of value columns exist
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[DVC / 8][4];
#pragma unroll
  for (int i = 0; i < DVC / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  for (int t = 0; t < stages; t++) {
    const int buf = t % NSTAGES;
    __syncthreads();                                  // every warp is done with the buffer before this one; cleared rows are visible
    if (s_failed) break;
    if (t + NSTAGES - 1 < stages) {
      const int ahead = (t + NSTAGES - 1) % NSTAGES;  // the buffer that was worked on last
      issue_stage<KEYS>(p, page_next, first + (t + NSTAGES - 1) * KEYS, sK + ahead * KEYS * stride, stride, &s_bar[ahead], tid);
      page_next = page_ahead<KEYS>(p, table, first + (t + NSTAGES) * KEYS, last, tid);
    }
    stage_landed(&s_bar[buf], (t / NSTAGES) & 1, p.status, &s_failed);
    const int key0 = first + t * KEYS + quarter * 16; // this warp's share of the stage
    if (key0 <= last && col0 < p.rank) {
      const __nv_bfloat16* tK = sK + (buf * KEYS + quarter * 16) * stride;
      float sc[2][4];
      if (shared_scores) {
        // the warps that hold the same keys (one per block of value columns) take a share of the rows' width each and add
        // their partial scores through shared memory
        const int k0 = steps * chunk / CHUNKS, k1 = steps * (chunk + 1) / CHUNKS;
        scores_block<2>(sQ, tK, stride, k0, k1, sc, lane);
        float4* mine = (float4*)s_part[warp];
        mine[lane] = make_float4(sc[0][0], sc[0][1], sc[0][2], sc[0][3]);
        mine[32 + lane] = make_float4(sc[1][0], sc[1][1], sc[1][2], sc[1][3]);
        asm volatile("bar.sync %0, %1;" ::"r"(1 + quarter), "r"(CHUNKS * 32) : "memory");
        // every warp adds the shares in the same order, its own among them: all of them hold the same scores, bit for bit
#pragma unroll
        for (int j = 0; j < 4; j++) sc[0][j] = sc[1][j] = 0.f;
#pragma unroll
        for (int from = 0; from < CHUNKS; from++) {
          const float4* share = (const float4*)s_part[from * PARTS + quarter];
          const float4 u = share[lane], v = share[32 + lane];
          sc[0][0] += u.x; sc[0][1] += u.y; sc[0][2] += u.z; sc[0][3] += u.w;
          sc[1][0] += v.x; sc[1][1] += v.y; sc[1][2] += v.z; sc[1][3] += v.w;
        }
      } else {
        scores_block<2>(sQ, tK, stride, 0, steps, sc, lane);
      }
      softmax_values_block<DVC, 2>(sc, tK, stride, col0, col_end, key0, last, last, key0 + 15 > last, scale_log2, m0, m1, l0, l1,
                                   o, lane);
    }
  }
  __syncthreads();                                    // every warp is done with the stages: they become the exchange area
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  float* so = (float*)sK;                             // [CHUNKS][PARTS][16 rows][DVC]
  if (qc == 0 && chunk == 0) {                        // every block of columns saw the same scores
    s_ml[quarter][gr][0] = m0 == -INFINITY ? -INFINITY : m0 * p.scale; s_ml[quarter][gr][1] = l0;
    s_ml[quarter][gr + 8][0] = m1 == -INFINITY ? -INFINITY : m1 * p.scale; s_ml[quarter][gr + 8][1] = l1;
  }
#pragma unroll
  for (int i = 0; i < DVC / 8; i++) {
    *(float2*)(so + ((warp * 16 + gr) * DVC) + i * 8 + qc * 2) = make_float2(o[i][0], o[i][1]);
    *(float2*)(so + ((warp * 16 + gr + 8) * DVC) + i * 8 + qc * 2) = make_float2(o[i][2], o[i][3]);
  }
  __syncthreads();
  const int cols = cta_col_end - cta_col0;
  for (int idx = tid; idx < 16 * cols; idx += THREADS) {
    const int row = idx / cols, c = idx % cols;
    if (head0 + row >= p.heads) continue;
    float top = -INFINITY;
#pragma unroll
    for (int w = 0; w < PARTS; w++) top = fmaxf(top, s_ml[w][row][0]);
    float sum = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < PARTS; w++) {
      const float f = s_ml[w][row][0] == -INFINITY ? 0.f : expf(s_ml[w][row][0] - top);
      sum = fmaf(f, so[(((c / DVC) * PARTS + w) * 16 + row) * DVC + c % DVC], sum);
      l = fmaf(f, s_ml[w][row][1], l);
    }
    const size_t at = ((size_t)r * p.splits + split) * p.heads + head0 + row;
    p.part_o[at * p.rank + cta_col0 + c] = sum;
    if (c == 0 && blockIdx.y == 0) { p.part_ml[at * 2] = top; p.part_ml[at * 2 + 1] = l; }
  }
}

// One block per (request, head): the ranges' partial sums and the sink become the output row.  The ranges' weights
// exp(m_s - top) / denominator are made once (shared memory, up to 64 ranges), then every column is one pass of
// independent loads.
__global__ void __launch_bounds__(128)
latent_attention_merge_kernel(const LatentParams p) {
  __shared__ float s_m[64], s_w[64];
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const size_t base = ((size_t)r * p.splits) * p.heads + h;
  if (tid < p.splits) s_m[tid] = p.part_ml[(base + (size_t)tid * p.heads) * 2];
  __syncthreads();
  float top = p.sink ? p.sink[h] : -INFINITY;
  for (int s = 0; s < p.splits; s++) top = fmaxf(top, s_m[s]);
  if (tid < p.splits) s_w[tid] = s_m[tid] == -INFINITY ? 0.f : expf(s_m[tid] - top);
  __syncthreads();
  float denom = p.sink ? expf(p.sink[h] - top) : 0.f;
  if (tid < 32) {
    float part = 0.f;
    for (int s = tid; s < p.splits; s += 32) part = fmaf(s_w[s], p.part_ml[(base + (size_t)s * p.heads) * 2 + 1], part);
    part = warp_sum(part);
    if (tid == 0) s_m[0] = denom + part;
  }
  __syncthreads();
  const float inv = 1.0f / s_m[0];
  const int token = p.q_start[r];
  for (int c = tid; c < p.rank; c += blockDim.x) {
    float sum = 0.f;
#pragma unroll 4
    for (int s = 0; s < p.splits; s++) sum = fmaf(s_w[s], p.part_o[(base + (size_t)s * p.heads) * p.rank + c], sum);
    p.out[((size_t)token * p.heads + h) * p.rank + c] = __float2bfloat16_rn(sum * inv);
  }
}

// dynamic bytes a CTA may ask for beside the kernels' static arrays (the split kernel's hold the warps' partial scores)
constexpr size_t ROWS_LIMIT = 232448 - 2048, SPLIT_LIMIT = 232448 - 18432;

// Raise a kernel's dynamic shared memory limit to what the SM has left beside the kernel's static arrays (once per
// kernel), and refuse a launch that wants more.
template <typename K>
int prepare(K kernel, size_t smem) {
  static thread_local const void* done[32];
  static thread_local size_t room[32];
  static thread_local int count = 0;
  for (int i = 0; i < count; i++)
    if (done[i] == (const void*)kernel)
      return smem <= room[i] ? 0 : sprout_fail("latent_attention: %zu bytes of shared memory wanted, %zu available", smem, room[i]);
  cudaFuncAttributes attributes;
  if (cudaFuncGetAttributes(&attributes, kernel) != cudaSuccess) return sprout_fail("latent_attention: cannot read the kernel's attributes");
  const size_t available = 232448 - attributes.sharedSizeBytes;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)available) != cudaSuccess)
    return sprout_fail("latent_attention: cannot raise the kernel's shared memory limit");
  if (count < 32) { done[count] = (const void*)kernel; room[count++] = available; }
  return smem <= available ? 0 : sprout_fail("latent_attention: %zu bytes of shared memory wanted, %zu available", smem, available);
}

// How a latent of `rank` columns is divided: DVC columns per warp, `chunks` such blocks per CTA, CTAs along y.
struct Division { int dvc, chunks, ctas; };
inline Division divide(int rank) {
  if (rank <= 128) return {128, 1, 1};
  if (rank <= 256) return {256, 1, 1};
  return {256, 2, (rank + 511) / 512};
}
// The split-key kernel takes blocks of 128 columns (half the accumulator registers, twice the warps an SM holds).
inline Division divide_split(int rank) {
  if (rank <= 128) return {128, 1, 1};
  if (rank <= 256) return {128, 2, 1};
  return {128, 4, (rank + 511) / 512};
}

}  // namespace

// Whether the tensor-core kernels take these sizes (else the caller runs the float32-arithmetic kernel).
SPROUT_API int sprout_latent_attention_mma_supported(int width, int rank) {
  if (width % 16 || rank % 16 || rank <= 0 || width < rank) return 0;
  const size_t row_bytes = (size_t)(width + 8) * 2;
  const int rows = 16 * WARPS / divide(rank).chunks;
  return (rows + 2 * 32) * row_bytes + (divide(rank).chunks == 2 ? 32 * 512 : 0) <= ROWS_LIMIT && (16 + 2 * 64) * row_bytes <= SPLIT_LIMIT;
}

// splits == 0: whole rows (any mix of portions and single tokens).  splits >= 1: every request brings one token
// and its keys are divided into `splits` ranges of `split_keys` keys (a multiple of 64 fills whole stages); `scratch` then holds
// requests * splits * heads * (rank + 2) floats.
SPROUT_API int sprout_latent_attention_mma(const void* q, const void* cache, const int* block_table, int table_stride,
                                           const int* q_start, const int* positions, const int* context_lens,
                                           const float* sink, void* out, float* scratch, int tokens, int requests,
                                           int heads, int width, int rank, int page_tokens, int num_pages, int splits,
                                           int split_keys, float scale, int* status, cudaStream_t stream) {
  SPROUT_REQUIRE(q && cache && block_table && q_start && positions && out && status, "latent_attention_mma: null pointer");
  SPROUT_REQUIRE(tokens > 0 && requests > 0 && heads > 0 && page_tokens > 0 && num_pages > 0 && scale > 0.f,
                 "latent_attention_mma: sizes and scale must be positive");
  SPROUT_REQUIRE(sprout_latent_attention_mma_supported(width, rank),
                 "latent_attention_mma: width (%d) and latent size (%d) must be multiples of 16 that fit shared memory", width, rank);
  LatentParams p;
  p.q = (const __nv_bfloat16*)q; p.cache = (const __nv_bfloat16*)cache; p.block_table = block_table; p.table_stride = table_stride;
  p.q_start = q_start; p.positions = positions; p.context_lens = context_lens; p.sink = sink; p.out = (__nv_bfloat16*)out;
  p.requests = requests; p.heads = heads; p.width = width; p.rank = rank; p.page_tokens = page_tokens; p.num_pages = num_pages;
  p.split_keys = split_keys; p.splits = splits; p.scale = scale; p.status = status;
  p.part_o = scratch; p.part_ml = scratch ? scratch + (size_t)requests * splits * heads * rank : nullptr;
  const Division d = divide(rank);
  const size_t row_bytes = (size_t)(width + 8) * 2;
  if (splits == 0) {
    const int rows = 16 * WARPS / d.chunks;
    const long long tiles = ((long long)tokens * heads + rows - 1) / rows + requests;
    SPROUT_REQUIRE(tiles <= 0x7fffffffLL, "latent_attention_mma: too many rows");
    // stages of 64 keys where they fit, else 32; with two blocks of value columns 48 or 32 (the partial scores of 8 warps
    // take KEYS x 512 bytes of static shared memory)
    const bool keys64 = d.chunks == 1 && (rows + 2 * 64) * row_bytes <= ROWS_LIMIT;
    const bool keys48 = d.chunks == 2 && (rows + 2 * 48) * row_bytes + 48 * 512 <= ROWS_LIMIT;
    const size_t smem = (rows + 2 * (keys64 ? 64 : keys48 ? 48 : 32)) * row_bytes;
    dim3 grid((unsigned)tiles, d.ctas);
#define LAUNCH_ROWS(DVC, KEYS, CHUNKS)                                                                              \
    do {                                                                                                            \
      if (prepare(latent_attention_rows_kernel<DVC, KEYS, CHUNKS>, smem)) return 1;                                       \
      sprout_launch(latent_attention_rows_kernel<DVC, KEYS, CHUNKS>, grid, dim3(WARPS * 32), smem, stream, p);      \
    } while (0)
    if (d.dvc == 128) { if (keys64) LAUNCH_ROWS(128, 64, 1); else LAUNCH_ROWS(128, 32, 1); }
    else if (d.chunks == 1) { if (keys64) LAUNCH_ROWS(256, 64, 1); else LAUNCH_ROWS(256, 32, 1); }
    else { if (keys48) LAUNCH_ROWS(256, 48, 2); else LAUNCH_ROWS(256, 32, 2); }
#undef LAUNCH_ROWS
    return sprout_check_launch("latent_attention_rows");
  }
  SPROUT_REQUIRE(splits <= 64, "latent_attention_mma: at most 64 ranges of keys (got %d)", splits);
  SPROUT_REQUIRE(tokens == requests && context_lens && scratch && split_keys > 0,
                 "latent_attention_mma: split keys need one token per request, context lengths, scratch and a positive number of keys per range");
  // Two stages of 64 keys, four warps per block of 128 value columns, up to four blocks (16 warps) per CTA.  (Measured
  // against it: three stages, of 64 keys or for wide rows of 48 keys with three warps per block, were slower, 91 against
  // 71 us at 64 requests of 2,048 keys and rows of 576: the kernel follows its warps' instruction chains, and larger CTAs
  // leave an SM fewer warps.)  The stages' room is used again for the warps' partial sums: [chunks][4][16][128] floats.
  const Division ds = divide_split(rank);
  const size_t exchange = (size_t)ds.chunks * 4 * 16 * ds.dvc * sizeof(float);
  const size_t smem = 16 * row_bytes + (2 * 64 * row_bytes > exchange ? 2 * 64 * row_bytes : exchange);
  SPROUT_REQUIRE(smem <= SPLIT_LIMIT, "latent_attention_mma: rows too wide for the split kernel's shared memory");
  dim3 grid(requests * ((heads + 15) / 16), ds.ctas, splits);
#define LAUNCH_SPLIT(DVC, CHUNKS, PARTS, NSTAGES)                                                                          \
  do {                                                                                                                     \
    if (prepare(latent_attention_split_kernel<DVC, CHUNKS, PARTS, NSTAGES>, smem)) return 1;                               \
    sprout_launch(latent_attention_split_kernel<DVC, CHUNKS, PARTS, NSTAGES>, grid, dim3(CHUNKS * PARTS * 32), smem, stream, p); \
  } while (0)
  if (ds.chunks == 1) LAUNCH_SPLIT(128, 1, 4, 2);
  else if (ds.chunks == 2) LAUNCH_SPLIT(128, 2, 4, 2);
  else LAUNCH_SPLIT(128, 4, 4, 2);
#undef LAUNCH_SPLIT
  if (int code = sprout_check_launch("latent_attention_split")) return code;
  sprout_launch(latent_attention_merge_kernel, dim3(requests, heads), dim3(128), 0, stream, p);
  return sprout_check_launch("latent_attention_merge");
}
