// Latent attention: every token keeps ONE vector in the cache, its normed latent c (R numbers) followed by one
// rotated key part k_r (P numbers) that all heads share; keys and values of the heads are linear in c:
//   k_h = U_h c,  v_h = V_h c,  score_h(i, j) = (q_h(i) . U_h c(j) + q_r,h(i) . k_r(j)) * scale.
// The kernels here work in the latent space: with a_h(i) = U_h^T q_h(i) (a product of the caller) the score is
// [a_h(i) ; q_r,h(i)] . [c(j) ; k_r(j)], and the weighted sum of the c(j) is multiplied by V_h afterwards (again a
// product of the caller).  So all heads of a token attend to the same rows of D_K = R + P numbers, and the values
// are the first R of them.
//
//   ms_latent_prepare            norm of c, rotation of k_r and of the queries' rotated parts, append to the cache
//   ms_latent_attention_generic  paged attention over such rows, float32 arithmetic, any sizes
//   ms_head_gate                 the heads' outputs times sigmoid(gate logit of the head)
#include "common.cuh"

namespace ms {

constexpr int kLatWarps = 4;
constexpr int kLatMaxLanes = 32;   // value lanes per thread: R up to 1024

// Rotation of element c of a vector of `rot` entries whose first `dims` are rotated: entry j < dims / 2 is paired
// with entry j + dims / 2; the table holds (cos, sin) of the token for each pair (already times the magnitude).
template <typename T>
__device__ __forceinline__ float rotated(const T* src, int c, int dims, const float2* table) {
  const float v = to_float(src[c]);
  if (c >= dims) return v;
  const int half = dims >> 1;
  const bool low = c < half;
  const float2 cs = table[low ? c : c - half];
  const float partner = to_float(src[low ? c + half : c - half]);
  return low ? v * cs.x - partner * cs.y : v * cs.x + partner * cs.y;
}

// One warp per (token, item): items 0 .. H-1 are the query heads, item H is the token's cache row.
//   head h: q_full[n, h, R + c] = rotate(q[n, h, dim + c])                 for c < P   (the unrotated part is the caller's)
//   row:    cache[slot, c] = w[c] * x[c] / sqrt(mean(x^2) + eps)           for c < R,  x = dkv[n, :R]
//           cache[slot, R + c] = rotate(dkv[n, R + c])                     for c < P
// `proj` holds a token's projections side by side: q heads from column q_col, [dkv] from column dkv_col.
template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ proj, int ld, int q_col, int dkv_col, int heads, int dim, int rot,
                                      int rank, const int* __restrict__ slots, const void* __restrict__ norm_weight,
                                      int weight_dtype, float eps, const float2* __restrict__ cos_sin, int rot_dims,
                                      T* __restrict__ cache, T* __restrict__ q_full, int n_tokens) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
  if (item >= (long long)n_tokens * (heads + 1)) return;
  const int n = (int)(item / (heads + 1)), which = (int)(item % (heads + 1));
  const float2* table = cos_sin + (size_t)n * (rot_dims >> 1);
  const int dk = rank + rot;
  if (which < heads) {
    const T* src = proj + (size_t)n * ld + q_col + (size_t)which * (dim + rot) + dim;
    T* dst = q_full + ((size_t)n * heads + which) * dk + rank;
    for (int c = lane; c < rot; c += 32) dst[c] = from_float<T>(rotated(src, c, rot_dims, table));
    return;
  }
  const int slot = slots[n];
  if (slot < 0) return;
  const T* src = proj + (size_t)n * ld + dkv_col;
  T* dst = cache + (size_t)slot * dk;
  float sum_sq = 0.f;
  for (int c = lane; c < rank; c += 32) {
    const float v = to_float(src[c]);
    sum_sq += v * v;
  }
  sum_sq = warp_sum(sum_sq);
  const float inv = 1.0f / sqrtf(sum_sq / (float)rank + eps);
  for (int c = lane; c < rank; c += 32)
    dst[c] = from_float<T>(load_as_float(norm_weight, weight_dtype, c) * (to_float(src[c]) * inv));
  for (int c = lane; c < rot; c += 32) dst[rank + c] = from_float<T>(rotated(src + rank, c, rot_dims, table));
}

__device__ __forceinline__ float latent_dot(const float* q_s, const float* row, int d) {
  float dot = 0.f;
  if ((d & 3) == 0) {
    for (int c = 0; c < d; c += 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + c);
      dot += q_s[c] * v.x;
      dot += q_s[c + 1] * v.y;
      dot += q_s[c + 2] * v.z;
      dot += q_s[c + 3] * v.w;
    }
  } else {
    for (int c = 0; c < d; ++c) dot += q_s[c] * row[c];
  }
  return dot;
}

__device__ __forceinline__ float latent_dot(const float* q_s, const __nv_bfloat16* row, int d) {
  float dot = 0.f;
  if ((d & 7) == 0) {
    for (int c = 0; c < d; c += 8) {
      const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 f = __bfloat1622float2(pairs[i]);
        dot += q_s[c + 2 * i] * f.x;
        dot += q_s[c + 2 * i + 1] * f.y;
      }
    }
  } else {
    for (int c = 0; c < d; ++c) dot += q_s[c] * __bfloat162float(row[c]);
  }
  return dot;
}

// One block of four warps per (token, head), as in the general key/value kernel: keys in blocks of 32 that start at
// absolute key 0, warp w takes blocks w, w + 4, ...; a lane scores one key (a serial dot product over D_K), the warp
// keeps a running maximum and sum, then every lane accumulates its lanes of the first R numbers of the 32 rows.  The
// four partial results are merged in warp order, so a token's result depends on its own position only.
template <typename T>
__global__ void latent_attention_generic_kernel(const T* __restrict__ q_full, const T* __restrict__ cache,
                                                const int* __restrict__ block_tables, int table_stride,
                                                const int* __restrict__ request_of_token, const int* __restrict__ positions,
                                                int page_size, int heads, int dk, int dv, float scale, int window,
                                                T* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float smem[];
  float* q_s = smem;                                  // [dk]
  float* part_acc = smem + dk;                        // [warps][dv]
  float* part_m = part_acc + kLatWarps * dv;          // [warps]
  float* part_l = part_m + kLatWarps;                 // [warps]

  const int token = blockIdx.x, head = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[token];
  const int* table = block_tables + (size_t)request_of_token[token] * table_stride;
  const T* q_row = q_full + ((size_t)token * heads + head) * dk;
  for (int c = threadIdx.x; c < dk; c += blockDim.x) q_s[c] = to_float(q_row[c]) * scale;
  __syncthreads();

  const int first_key = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int last_key = pos;  // inclusive
  float m = -INFINITY, l = 0.f;
  float acc[kLatMaxLanes];
#pragma unroll
  for (int i = 0; i < kLatMaxLanes; ++i) acc[i] = 0.f;

  const int first_block = first_key / 32, last_block = last_key / 32;
  for (int block = first_block + ((warp - first_block % kLatWarps + kLatWarps) % kLatWarps); block <= last_block;
       block += kLatWarps) {
    const int key = block * 32 + lane;
    const bool valid = key >= first_key && key <= last_key;
    float score = -INFINITY;
    size_t row_offset = 0;
    if (valid) {
      const int page = table[key / page_size];
      row_offset = ((size_t)page * page_size + key % page_size) * dk;
      score = latent_dot(q_s, cache + row_offset, dk);
    }
    const float block_max = warp_max(score);
    const float new_m = fmaxf(m, block_max);       // finite: every block holds at least one valid key
    const float correction = expf(m - new_m);      // m == -inf on the first block gives 0
    const float p = valid ? expf(score - new_m) : 0.f;
    l = l * correction + warp_sum(p);
    m = new_m;
#pragma unroll
    for (int i = 0; i < kLatMaxLanes; ++i) acc[i] *= correction;
    for (int j = 0; j < 32; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t off_j = __shfl_sync(0xffffffffu, (unsigned long long)row_offset, j);
      if (pj == 0.f) continue;   // uniform across the warp
      const T* v_row = cache + off_j;
#pragma unroll
      for (int i = 0; i < kLatMaxLanes; ++i) {
        const int c = lane + 32 * i;
        if (c < dv) acc[i] += pj * to_float(v_row[c]);
      }
    }
  }

  if (lane == 0) {
    part_m[warp] = m;
    part_l[warp] = l;
  }
#pragma unroll
  for (int i = 0; i < kLatMaxLanes; ++i) {
    const int c = lane + 32 * i;
    if (c < dv) part_acc[warp * dv + c] = acc[i];
  }
  __syncthreads();
  float m_all = -INFINITY;
  for (int w = 0; w < kLatWarps; ++w) m_all = fmaxf(m_all, part_m[w]);
  float l_all = 0.f;
  for (int w = 0; w < kLatWarps; ++w) l_all += part_m[w] == -INFINITY ? 0.f : part_l[w] * expf(part_m[w] - m_all);
  T* out_row = out + ((size_t)token * heads + head) * dv;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float sum = 0.f;
    for (int w = 0; w < kLatWarps; ++w)
      if (part_m[w] != -INFINITY) sum += part_acc[w * dv + c] * expf(part_m[w] - m_all);
    out_row[c] = from_float<T>(sum / l_all);
  }
}

// x[n, h, :] *= sigmoid(gate[n * ld + h])
template <typename T>
__global__ void head_gate_kernel(T* __restrict__ x, const T* __restrict__ gate, int ld, int heads, int vdim, size_t total) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t row = i / vdim;                  // n * heads + h
  const size_t n = row / heads;
  const int h = (int)(row % heads);
  const float g = to_float(gate[n * ld + h]);
  x[i] = from_float<T>(to_float(x[i]) / (1.0f + expf(-g)));
}

}  // namespace ms

using namespace ms;

#define MS_LAT_DISPATCH(dtype, ...)                              \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

// proj [n_tokens, ld]: q heads ([dim unrotated, rot rotated] each) from column q_col, the down-projection
// ([rank latent, rot rotated key part]) from column dkv_col; cache [rows, rank + rot]; q_full [n_tokens, heads, rank + rot]
// (its first `rank` numbers per head are not touched); cos_sin float32 [n_tokens, rot_dims / 2, 2] or null with rot_dims 0.
MS_EXPORT int ms_latent_prepare(const void* proj, int dtype, int ld, int q_col, int dkv_col, int heads, int dim, int rot,
                                int rank, const int* slots, const void* norm_weight, int weight_dtype, float eps,
                                const float* cos_sin, int rot_dims, void* cache, void* q_full, int n_tokens,
                                cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(heads > 0 && dim >= 0 && rot >= 0 && rank > 0, "latent_prepare: sizes must be positive (heads %d dim %d rot %d rank %d)",
             heads, dim, rot, rank);
  MS_REQUIRE(rot_dims >= 0 && rot_dims <= rot && rot_dims % 2 == 0,
             "latent_prepare: %d rotated dimensions must be even and at most the rotated part %d", rot_dims, rot);
  MS_REQUIRE(rot_dims == 0 || cos_sin != nullptr, "latent_prepare: a rotation needs its table");
  const int warps = 4;
  const long long items = (long long)n_tokens * (heads + 1);
  const long long blocks = (items + warps - 1) / warps;
  MS_REQUIRE(blocks < 2147483647LL, "latent_prepare: %lld items in one launch is too many", items);
  MS_LAT_DISPATCH(dtype, (ms::launch(latent_prepare_kernel<T>, (unsigned)blocks, warps * 32, 0, stream, (const T*)proj, ld, q_col,
                                     dkv_col, heads, dim, rot, rank, slots, norm_weight, weight_dtype, eps,
                                     (const float2*)cos_sin, rot_dims, (T*)cache, (T*)q_full, n_tokens)));
  MS_CHECK_LAUNCH("latent_prepare");
  return 0;
}

// q_full [n_tokens, heads, dk]; cache of one layer [pages, page_size, dk]; out [n_tokens, heads, dv] (dv <= dk: the
// values are the first dv numbers of a row).  A token at position p sees rows max(0, p - window + 1) .. p of its
// own request (window <= 0: all), which must be in the cache already.
MS_EXPORT int ms_latent_attention_generic(const void* q_full, int dtype, const void* cache, const int* block_tables,
                                          int table_stride, const int* request_of_token, const int* positions,
                                          int page_size, int heads, int dk, int dv, float scale, int window, void* out,
                                          int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(dv > 0 && dv <= dk && dv <= 32 * kLatMaxLanes, "latent_attention: value size %d outside 1..min(%d, %d)", dv, dk,
             32 * kLatMaxLanes);
  MS_REQUIRE(page_size > 0, "latent_attention: page size must be positive, got %d", page_size);
  MS_REQUIRE(heads > 0 && heads <= 65535, "latent_attention: %d heads outside 1..65535", heads);
  const size_t smem = (size_t)(dk + kLatWarps * dv + 2 * kLatWarps) * sizeof(float);
  MS_REQUIRE(smem <= 48 * 1024, "latent_attention: rows of %d numbers need %zu bytes of shared memory", dk, smem);
  dim3 grid(n_tokens, heads);
  MS_LAT_DISPATCH(dtype, (ms::launch(latent_attention_generic_kernel<T>, grid, kLatWarps * 32, smem, stream, (const T*)q_full,
                                     (const T*)cache, block_tables, table_stride, request_of_token, positions, page_size,
                                     heads, dk, dv, scale, window, (T*)out)));
  MS_CHECK_LAUNCH("latent_attention_generic");
  return 0;
}

// x [n_tokens, heads, vdim] in place; gate logits of token n at gate[n * ld + h].
MS_EXPORT int ms_head_gate(void* x, const void* gate, int dtype, int ld, int heads, int vdim, int n_tokens,
                           cudaStream_t stream) {
  const size_t total = (size_t)n_tokens * heads * vdim;
  if (total == 0) return 0;
  const size_t blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647ULL, "head_gate: %zu elements in one launch is too many", total);
  MS_LAT_DISPATCH(dtype, (ms::launch(head_gate_kernel<T>, (unsigned)blocks, 256, 0, stream, (T*)x, (const T*)gate, ld, heads, vdim,
                                     total)));
  MS_CHECK_LAUNCH("head_gate");
  return 0;
}
