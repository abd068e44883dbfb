// The selective state-space mixer: what lies between its input projection and its output projection.
//
//   ms_causal_conv_silu   per channel a causal convolution of a few taps with a bias, then SiLU, over the tokens of every
//                         request in the batch; the request's last (taps - 1) inputs are kept in its state vector
//   ms_selective_scan     per head S_t = exp(-exp(A_log) dt_t) S_(t-1) + dt_t B_t x_t^T and y_t = S_t^T C_t + D x_t with
//                         dt_t = softplus(dt_t + dt_bias), walked token by token from the state the request's slot holds
//   ms_gated_group_norm   out = weight * (y silu(z)) / rms(y silu(z)), the root mean square taken per group of channels
//
// Everything here is float32 arithmetic on float32 state; only the projection that the kernels read (z, the
// convolution's inputs, dt) and the last kernel's output are in the model's compute type.  A request's tokens are
// walked in order and every sum has a fixed order, so a position's result depends on the tokens before it alone, not
// on how they were cut into steps, on what else is in the batch or on which state slot the request holds.
//
// A request's state vector: [taps - 1][channels] convolution inputs, oldest first, then [heads][P][N] head states
// (zero at admission: the zeros before a sequence's start and the empty state are the same thing).
#include "common.cuh"

namespace ms {

constexpr int kConvTokens = 64;      // tokens of a request that one thread walks
constexpr int kMaxTaps = 8;

__device__ __forceinline__ float silu_f(float v) { return v / (1.f + expf(-v)); }

// grid (channel blocks, token chunks, requests); a thread owns one channel and walks kConvTokens tokens with the last
// inputs in registers.  The block of a request's FIRST chunk also writes the request's new convolution state: it is the
// only block that reads the old one (into registers, before anything is written), so nothing races.
template <typename T>
__global__ void __launch_bounds__(128)
causal_conv_silu_kernel(const T* __restrict__ proj, int ld, int col, int channels, int taps,
                        const float* __restrict__ weight, const float* __restrict__ bias, float* __restrict__ states,
                        long long state_stride, int state_offset, const int* __restrict__ state_slots,
                        const int* __restrict__ query_start, float* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int request = blockIdx.z;
  const int q0 = query_start[request], q_len = query_start[request + 1] - q0;
  const int t0 = blockIdx.y * kConvTokens;
  if (c >= channels || t0 >= q_len) return;
  float* state = states + (long long)state_slots[request] * state_stride + state_offset;     // [taps - 1][channels]
  const int keep = taps - 1;
  float w[kMaxTaps], window[kMaxTaps];       // window[k]: the input that tap k meets at the current token
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) w[k] = k < taps ? weight[(size_t)c * taps + k] : 0.f;
  const float b = bias[c];
  // inputs before token t0: from the batch where the request's portion reaches back that far, else from the state
  // (the input at local index i < 0 is state[keep + i])
#pragma unroll
  for (int k = 0; k < kMaxTaps; ++k) window[k] = 0.f;
#pragma unroll
  for (int k = 0; k + 1 < kMaxTaps; ++k) {
    if (k + 1 < taps) {                      // slots 1 .. taps - 1 hold inputs t0 - keep + k .. ; slot 0 is shifted out first
      const int i = t0 - keep + k;
      window[k + 1] = i >= 0 ? to_float(proj[(size_t)(q0 + i) * ld + col + c]) : state[(size_t)(keep + i) * channels + c];
    }
  }
  if (t0 == 0) {
    // new state: the last `keep` inputs of (old state, this portion)
    for (int j = 0; j < keep; ++j) {
      const int i = q_len - keep + j;        // local index of the input that becomes state[j]
      float v = 0.f;
      if (i >= 0) {
        v = to_float(proj[(size_t)(q0 + i) * ld + col + c]);
      } else {
#pragma unroll
        for (int k = 1; k < kMaxTaps; ++k)
          if (k == 1 + keep + i) v = window[k];      // = old state[keep + i], read above, before this write
      }
      state[(size_t)j * channels + c] = v;
    }
  }
  const int t_end = min(q_len, t0 + kConvTokens);
  for (int t = t0; t < t_end; ++t) {
#pragma unroll
    for (int k = 0; k + 1 < kMaxTaps; ++k) window[k] = window[k + 1];
    // after the shift the newest input belongs at index taps - 1
    const float u = to_float(proj[(size_t)(q0 + t) * ld + col + c]);
    float sum = b;
#pragma unroll
    for (int k = 0; k < kMaxTaps; ++k) {
      if (k == taps - 1) window[k] = u;
      if (k < taps) sum += w[k] * window[k];
    }
    out[(size_t)(q0 + t) * channels + c] = silu_f(sum);
  }
}

// The recurrence.  grid (column blocks of a head, heads, requests); a block of 128 threads owns 16 channels (columns p) of
// one head of one request: 8 lanes per column, lane j holding the state entries n = j, j + 8, ... (R of them) in
// registers.  Tokens are staged through shared memory in chunks; y_t[p] is the lanes' partial sums added by a fixed tree.
constexpr int kScanLanes = 8, kScanColumns = 16, kScanChunk = 16;

template <typename T, int R>
__global__ void __launch_bounds__(kScanLanes * kScanColumns)
selective_scan_kernel(const float* __restrict__ conv, int conv_ld, const T* __restrict__ proj, int ld, int dt_col,
                      const float* __restrict__ dt_bias, const float* __restrict__ a_log, const float* __restrict__ d_skip,
                      float* __restrict__ states, long long state_stride, int state_offset,
                      const int* __restrict__ state_slots, const int* __restrict__ query_start, int heads, int P, int N,
                      int groups, float* __restrict__ y) {
  grid_dependency_wait();
  grid_dependency_launch();
  extern __shared__ float scan_smem[];
  float* b_s = scan_smem;                         // [chunk][N]
  float* c_s = b_s + kScanChunk * N;              // [chunk][N]
  float* x_s = c_s + kScanChunk * N;              // [chunk][columns]
  float* dt_s = x_s + kScanChunk * kScanColumns;  // [chunk]: step size
  float* decay_s = dt_s + kScanChunk;             // [chunk]
  const int head = blockIdx.y, request = blockIdx.z;
  const int p0 = blockIdx.x * kScanColumns;
  const int tid = threadIdx.x, lane = tid % kScanLanes, column = tid / kScanLanes;
  const int p = p0 + column;
  const int q0 = query_start[request], q_len = query_start[request + 1] - q0;
  if (q_len <= 0) return;
  const int group = head / (heads / groups);
  const int inner = heads * P;
  float* state = states + (long long)state_slots[request] * state_stride + state_offset + ((size_t)head * P + p) * N;
  float s[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int n = lane + kScanLanes * i;
    s[i] = (p < P && n < N) ? state[n] : 0.f;
  }
  const float a = -expf(a_log[head]);
  const float bias = dt_bias[head], skip = d_skip[head];
  for (int t0 = 0; t0 < q_len; t0 += kScanChunk) {
    const int count = min(kScanChunk, q_len - t0);
    __syncthreads();
    for (int i = tid; i < count * N; i += blockDim.x) {
      const int t = i / N, n = i % N;
      const float* row = conv + (size_t)(q0 + t0 + t) * conv_ld + inner + group * N + n;
      b_s[t * N + n] = row[0];
      c_s[t * N + n] = row[(size_t)groups * N];
    }
    for (int i = tid; i < count * kScanColumns; i += blockDim.x) {
      const int t = i / kScanColumns, cc = i % kScanColumns;
      x_s[i] = p0 + cc < P ? conv[(size_t)(q0 + t0 + t) * conv_ld + head * P + p0 + cc] : 0.f;
    }
    if (tid < count) {
      const float raw = to_float(proj[(size_t)(q0 + t0 + tid) * ld + dt_col + head]) + bias;
      const float step = raw > 20.f ? raw : log1pf(expf(raw));        // softplus; above 20 the two agree in float32
      dt_s[tid] = step;
      decay_s[tid] = expf(a * step);
    }
    __syncthreads();
    for (int t = 0; t < count; ++t) {
      const float decay = decay_s[t], xv = x_s[t * kScanColumns + column], in = dt_s[t] * xv;
      float partial = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        const int n = lane + kScanLanes * i;
        if (n < N) {
          s[i] = decay * s[i] + in * b_s[t * N + n];
          partial += s[i] * c_s[t * N + n];
        }
      }
      partial += __shfl_xor_sync(0xffffffffu, partial, 1);
      partial += __shfl_xor_sync(0xffffffffu, partial, 2);
      partial += __shfl_xor_sync(0xffffffffu, partial, 4);
      if (lane == 0 && p < P) y[(size_t)(q0 + t0 + t) * inner + head * P + p] = partial + skip * xv;
    }
  }
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int n = lane + kScanLanes * i;
    if (p < P && n < N) state[n] = s[i];
  }
}

// One block per (token, group): v = y * silu(z); out = weight * v / sqrt(mean(v^2) + eps).
template <typename T>
__global__ void gated_group_norm_kernel(const float* __restrict__ y, const T* __restrict__ proj, int ld, int z_col,
                                        const float* __restrict__ weight, int groups, int inner, float eps,
                                        T* __restrict__ out) {
  grid_dependency_wait();
  grid_dependency_launch();
  __shared__ float scratch[32];
  const size_t token = blockIdx.x;
  const int size = inner / groups, c0 = blockIdx.y * size;
  float sum_sq = 0.f;
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    const float v = y[token * inner + c0 + c] * silu_f(to_float(proj[token * ld + z_col + c0 + c]));
    sum_sq += v * v;
  }
  const float inv = 1.0f / sqrtf(block_sum(sum_sq, scratch) / (float)size + eps);
  for (int c = threadIdx.x; c < size; c += blockDim.x) {
    const float v = y[token * inner + c0 + c] * silu_f(to_float(proj[token * ld + z_col + c0 + c]));
    out[token * inner + c0 + c] = from_float<T>(v * inv * weight[c0 + c]);
  }
}

}  // namespace ms

using namespace ms;

#define MS_SS_DISPATCH(dtype, ...)                               \
  if ((dtype) == MS_F32) { using T = float; __VA_ARGS__; }       \
  else if ((dtype) == MS_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
  else MS_FAIL("unknown element type code %d", (dtype));

// proj [tokens, ld]: the convolution's inputs are its columns col .. col + channels; weight float32 [channels, taps] (the
// last tap is the current token's), bias float32 [channels]; states float32, one row of state_stride numbers per slot,
// the convolution's part at state_offset; out float32 [tokens, channels].
MS_EXPORT int ms_causal_conv_silu(const void* proj, int dtype, int ld, int col, int channels, int taps, const float* weight,
                                  const float* bias, float* states, long long state_stride, int state_offset,
                                  const int* state_slots, const int* query_start, int n_requests, int max_query_len,
                                  float* out, cudaStream_t stream) {
  if (n_requests == 0 || max_query_len == 0 || channels == 0) return 0;
  MS_REQUIRE(taps >= 1 && taps <= kMaxTaps, "causal_conv_silu: %d taps outside 1..%d", taps, kMaxTaps);
  const int chunks = (max_query_len + kConvTokens - 1) / kConvTokens;
  MS_REQUIRE(chunks <= 65535 && n_requests <= 65535, "causal_conv_silu: grid %d x %d exceeds the launch limits", chunks, n_requests);
  dim3 grid((channels + 127) / 128, chunks, n_requests);
  MS_SS_DISPATCH(dtype, (ms::launch(causal_conv_silu_kernel<T>, grid, 128, 0, stream, (const T*)proj, ld, col, channels, taps,
                                    weight, bias, states, state_stride, state_offset, state_slots, query_start, out)));
  MS_CHECK_LAUNCH("causal_conv_silu");
  return 0;
}

MS_EXPORT int ms_scan_max_state() { return kScanLanes * 32; }

// conv float32 [tokens, conv_ld] = [x: heads * P | B: groups * N | C: groups * N]; dt is column dt_col + head of proj;
// dt_bias, a_log, d float32 [heads]; the heads' states [heads][P][N] at state_offset of a slot's row; y float32
// [tokens, heads * P].
MS_EXPORT int ms_selective_scan(const float* conv, int conv_ld, const void* proj, int dtype, int ld, int dt_col,
                                const float* dt_bias, const float* a_log, const float* d, float* states,
                                long long state_stride, int state_offset, const int* state_slots, const int* query_start,
                                int n_requests, int heads, int p, int n_state, int groups, float* y, cudaStream_t stream) {
  if (n_requests == 0) return 0;
  MS_REQUIRE(heads > 0 && groups > 0 && heads % groups == 0, "selective_scan: %d heads in %d groups", heads, groups);
  MS_REQUIRE(n_state >= 1 && n_state <= kScanLanes * 32, "selective_scan: a state of %d numbers per channel outside 1..%d",
             n_state, kScanLanes * 32);
  MS_REQUIRE(heads <= 65535 && n_requests <= 65535, "selective_scan: grid exceeds the launch limits");
  dim3 grid((p + kScanColumns - 1) / kScanColumns, heads, n_requests);
  const size_t smem = (size_t)(2 * kScanChunk * n_state + kScanChunk * kScanColumns + 2 * kScanChunk) * sizeof(float);
  const int per_lane = (n_state + kScanLanes - 1) / kScanLanes;
#define MS_SCAN(R)                                                                                                          \
  MS_SS_DISPATCH(dtype, (ms::launch(selective_scan_kernel<T, R>, grid, kScanLanes * kScanColumns, smem, stream, conv, conv_ld, \
                                    (const T*)proj, ld, dt_col, dt_bias, a_log, d, states, state_stride, state_offset,       \
                                    state_slots, query_start, heads, p, n_state, groups, y)))
  if (per_lane <= 2) { MS_SCAN(2); } else if (per_lane <= 4) { MS_SCAN(4); } else if (per_lane <= 8) { MS_SCAN(8); }
  else if (per_lane <= 16) { MS_SCAN(16); } else { MS_SCAN(32); }
#undef MS_SCAN
  MS_CHECK_LAUNCH("selective_scan");
  return 0;
}

// y float32 [tokens, inner]; z is columns z_col .. z_col + inner of proj [tokens, ld]; weight float32 [inner];
// out [tokens, inner] in proj's type.
MS_EXPORT int ms_gated_group_norm(const float* y, const void* proj, int dtype, int ld, int z_col, const float* weight,
                                  int groups, int inner, float eps, void* out, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0 || inner == 0) return 0;
  MS_REQUIRE(groups > 0 && inner % groups == 0 && groups <= 65535, "gated_group_norm: %d channels in %d groups", inner, groups);
  const int size = inner / groups;
  const int threads = size >= 1024 ? 256 : (size >= 256 ? 128 : 64);
  dim3 grid(n_tokens, groups);
  MS_SS_DISPATCH(dtype, (ms::launch(gated_group_norm_kernel<T>, grid, threads, 0, stream, y, (const T*)proj, ld, z_col, weight,
                                    groups, inner, eps, (T*)out)));
  MS_CHECK_LAUNCH("gated_group_norm");
  return 0;
}
