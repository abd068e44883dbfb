// A feed-forward of routed experts, on the device from the router to the weighted sum, so that a step never waits
// for the host to learn which experts were chosen (and a captured decode step can hold it):
//
//   ms_router_topk      float32 router logits W x + b of every token, the `top` largest, softmax over those alone
//   ms_expert_route     sorts the (token, choice) pairs by expert: segment offsets, the pairs in sorted order and
//                       each pair's place in that order
//   ms_expert_linear    one product per expert over its segment of rows (rows gathered from the tokens for the first
//                       product of an expert), optional squared-ReLU on the results
//   ms_expert_combine   out[token] = sum over its choices of weight * result row (+ a shared expert's output)
//   ms_relu_square      x = max(x, 0)^2 in place
//
// The products accumulate in float32 with one thread per output element summing k in ascending order, so a row's
// result does not depend on what else is in the batch or on where the row was sorted to.
#include "common.cuh"
#include "mma_common.cuh"

namespace ms {

// One warp per token.  logits[e] = sum_c x[c] W[e, c] + b[e] (lane-strided partial sums, then a fixed tree).  The
// `top` largest are taken one after the other (ties: the lower index); weights are exp(l - l_max) / sum over the taken.
template <typename T>
__global__ void router_topk_kernel(const T* __restrict__ x, const float* __restrict__ weight, const float* __restrict__ bias,
                                   int width, int experts, int top, int* __restrict__ ids, float* __restrict__ weights,
                                   int n_tokens) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float smem[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* logits = smem + (size_t)warp * (experts + top);
  float* taken = logits + experts;
  const int n = blockIdx.x * warps + warp;
  if (n >= n_tokens) return;
  const T* row = x + (size_t)n * width;
  for (int e = 0; e < experts; ++e) {
    const float* w = weight + (size_t)e * width;
    float sum = 0.f;
    for (int c = lane; c < width; c += 32) sum += to_float(row[c]) * w[c];
    sum = warp_sum(sum);
    if (lane == 0) logits[e] = sum + (bias ? bias[e] : 0.f);
  }
  __syncwarp();
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = logits[e];
      if (v > best) { best = v; best_e = e; }       // ascending e: the lower index wins a tie
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, best, o);
      const int other_e = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (other > best || (other == best && other_e < best_e)) { best = other; best_e = other_e; }
    }
    if (lane == 0) {
      taken[k] = best;
      ids[(size_t)n * top + k] = best_e;
      logits[best_e] = -INFINITY;
    }
    __syncwarp();
  }
  const float peak = taken[0];
  float total = 0.f;
  for (int k = 0; k < top; ++k) total += expf(taken[k] - peak);
  for (int k = lane; k < top; k += 32) weights[(size_t)n * top + k] = expf(taken[k] - peak) / total;
}

// One block.  offsets[e] .. offsets[e + 1] is expert e's segment of the sorted order; order[i] is the pair (token * top
// + choice) at place i, place[pair] its place.  Within a segment the order is arbitrary: rows are computed independently.
__global__ void expert_route_kernel(const int* __restrict__ ids, int pairs, int experts, int* __restrict__ offsets,
                                    int* __restrict__ order, int* __restrict__ place) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ int route_smem[];
  int* counts = route_smem;              // [experts]
  int* cursor = route_smem + experts;    // [experts]
  for (int e = threadIdx.x; e < experts; e += blockDim.x) counts[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&counts[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int running = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = running;
      cursor[e] = running;
      running += counts[e];
    }
    offsets[experts] = running;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int at = atomicAdd(&cursor[ids[i]], 1);
    order[at] = i;
    place[i] = at;
  }
}

constexpr int EBM = 64, EBN = 64, EBK = 16, ETM = 4, ETN = 4;

// C[i, :] = act(A[src(i), :] W_e^T) for every place i of expert e's segment; W [experts, N, K].  blockIdx.y walks the
// row tiles of all segments one after the other (a segment's last tile may be partial); tiles beyond the last do nothing.
// src(i) = order[i] / top with `order` (rows gathered from the tokens), else i.
template <typename T>
__global__ void __launch_bounds__(256)
expert_linear_kernel(const T* __restrict__ A, int lda, const int* __restrict__ order, int top, const T* __restrict__ W,
                     T* __restrict__ C, int ldc, const int* __restrict__ offsets, int experts, int N, int K, int relu_square) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float As[EBK][EBM + 4];
  __shared__ float Ws[EBK][EBN + 4];
  __shared__ int src_row[EBM];
  int tile = blockIdx.y, expert = 0, first = 0, end = 0;
  for (; expert < experts; ++expert) {
    first = offsets[expert];
    end = offsets[expert + 1];
    const int tiles = (end - first + EBM - 1) / EBM;
    if (tile < tiles) break;
    tile -= tiles;
  }
  if (expert == experts) return;
  const int m0 = first + tile * EBM, n0 = blockIdx.x * EBN;
  const int tid = threadIdx.x;
  if (tid < EBM) {
    const int i = m0 + tid;
    src_row[tid] = i < end ? (order ? order[i] / top : i) : -1;
  }
  __syncthreads();
  const T* We = W + (size_t)expert * N * K;
  const int tx = tid % 16, ty = tid / 16;
  const int load_row = tid / 4, load_k = (tid % 4) * 4;
  const int a_row = src_row[load_row];
  float acc[ETM][ETN] = {};
  for (int k0 = 0; k0 < K; k0 += EBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + load_k + i;
      const int wn = n0 + load_row;
      As[load_k + i][load_row] = (a_row >= 0 && k < K) ? to_float(A[(size_t)a_row * lda + k]) : 0.f;
      Ws[load_k + i][load_row] = (wn < N && k < K) ? to_float(We[(size_t)wn * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < EBK; ++k) {
      float a[ETM], w[ETN];
#pragma unroll
      for (int i = 0; i < ETM; ++i) a[i] = As[k][ty * ETM + i];
#pragma unroll
      for (int j = 0; j < ETN; ++j) w[j] = Ws[k][tx * ETN + j];
#pragma unroll
      for (int i = 0; i < ETM; ++i)
#pragma unroll
        for (int j = 0; j < ETN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < ETM; ++i) {
    const int m = m0 + ty * ETM + i;
    if (m >= end) continue;
#pragma unroll
    for (int j = 0; j < ETN; ++j) {
      const int n = n0 + tx * ETN + j;
      if (n >= N) continue;
      float v = acc[i][j];
      if (relu_square) { v = fmaxf(v, 0.f); v *= v; }
      C[(size_t)m * ldc + n] = from_float<T>(v);
    }
  }
}

// One block per token: out[n, c] = sum_k weights[n, k] * Y[place[n * top + k], c] (+ shared[n, c]), k ascending, float32.
template <typename T>
__global__ void expert_combine_kernel(const T* __restrict__ Y, int ldy, const int* __restrict__ place,
                                      const float* __restrict__ weights, int top, const T* __restrict__ shared,
                                      T* __restrict__ out, int width) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t n = blockIdx.x;
  for (int c = threadIdx.x; c < width; c += blockDim.x) {
    float sum = 0.f;
    for (int k = 0; k < top; ++k) sum += weights[n * top + k] * to_float(Y[(size_t)place[n * top + k] * ldy + c]);
    if (shared) sum += to_float(shared[n * width + c]);
    out[n * width + c] = from_float<T>(sum);
  }
}

template <typename T>
__global__ void relu_square_kernel(T* __restrict__ x, size_t total) {
  grid_dependency_wait();
  grid_dependency_launch();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const float v = fmaxf(to_float(x[i]), 0.f);
  x[i] = from_float<T>(v * v);
}

}  // namespace ms

using namespace ms;

#define MS_EXP_DISPATCH(dtype, ...)                              \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

// x [n_tokens, width]; weight float32 [experts, width]; bias float32 [experts] or null; ids int32 and weights float32
// [n_tokens, top].
MS_EXPORT int ms_router_topk(const void* x, int dtype, const float* weight, const float* bias, int width, int experts,
                             int top, int* ids, float* weights, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  MS_REQUIRE(experts > 0 && top > 0 && top <= experts, "router_topk: %d of %d experts", top, experts);
  const int warps = 4;
  const size_t smem = (size_t)warps * (experts + top) * sizeof(float);
  MS_REQUIRE(smem <= 48 * 1024, "router_topk: %d experts need %zu bytes of shared memory", experts, smem);
  MS_EXP_DISPATCH(dtype, (ms::launch(router_topk_kernel<T>, (n_tokens + warps - 1) / warps, warps * 32, smem, stream, (const T*)x,
                                     weight, bias, width, experts, top, ids, weights, n_tokens)));
  MS_CHECK_LAUNCH("router_topk");
  return 0;
}

// ids [pairs] (each in 0 .. experts - 1); offsets [experts + 1]; order, place [pairs].
MS_EXPORT int ms_expert_route(const int* ids, int pairs, int experts, int* offsets, int* order, int* place,
                              cudaStream_t stream) {
  MS_REQUIRE(experts > 0 && experts <= 4096, "expert_route: %d experts outside 1..4096", experts);
  ms::launch(expert_route_kernel, 1, 1024, (size_t)2 * experts * sizeof(int), stream, ids, pairs, experts, offsets, order, place);
  MS_CHECK_LAUNCH("expert_route");
  return 0;
}

// A rows of K numbers (row stride lda); order null or [pairs]; W [experts, N, K]; C [pairs, ldc].
MS_EXPORT int ms_expert_linear(const void* A, int dtype, int lda, const int* order, int top, const void* W, void* C, int ldc,
                               const int* offsets, int experts, int pairs, int N, int K, int relu_square, cudaStream_t stream) {
  if (pairs == 0 || N == 0) return 0;
  MS_REQUIRE(K > 0 && top > 0, "expert_linear: inner size %d and choices %d must be positive", K, top);
  const int row_tiles = (pairs + EBM - 1) / EBM + experts;      // every segment may end in a partial tile
  MS_REQUIRE(row_tiles <= 65535, "expert_linear: %d rows in one launch is too many", pairs);
  dim3 grid((N + EBN - 1) / EBN, row_tiles);
  MS_EXP_DISPATCH(dtype, (ms::launch(expert_linear_kernel<T>, grid, 256, 0, stream, (const T*)A, lda, order, top, (const T*)W,
                                     (T*)C, ldc, offsets, experts, N, K, relu_square)));
  MS_CHECK_LAUNCH("expert_linear");
  return 0;
}

// Y [pairs, ldy]; place [n_tokens * top]; weights float32 [n_tokens, top]; shared [n_tokens, width] or null; out [n_tokens, width].
MS_EXPORT int ms_expert_combine(const void* Y, int dtype, int ldy, const int* place, const float* weights, int top,
                                const void* shared, void* out, int width, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0 || width == 0) return 0;
  MS_EXP_DISPATCH(dtype, (ms::launch(expert_combine_kernel<T>, n_tokens, 256, 0, stream, (const T*)Y, ldy, place, weights, top,
                                     (const T*)shared, (T*)out, width)));
  MS_CHECK_LAUNCH("expert_combine");
  return 0;
}

MS_EXPORT int ms_relu_square(void* x, int dtype, long long total, cudaStream_t stream) {
  if (total <= 0) return 0;
  const long long blocks = (total + 255) / 256;
  MS_REQUIRE(blocks < 2147483647LL, "relu_square: %lld elements in one launch is too many", total);
  MS_EXP_DISPATCH(dtype, (ms::launch(relu_square_kernel<T>, (unsigned)blocks, 256, 0, stream, (T*)x, (size_t)total)));
  MS_CHECK_LAUNCH("relu_square");
  return 0;
}
