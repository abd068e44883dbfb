// Latent attention on the tensor cores (bfloat16, mma.sync.m16n8k16, float32 scores and sums).
//
// All heads of a token attend to the same cached rows [c ; k_r] of D_K numbers, whose first D_V numbers are also the
// values (attention_latent.cu), so a request's query rows (token-major, head-minor: row = token * H + head) form ONE
// matrix Q [tokens * H, D_K] against ONE key matrix K [context, D_K] and value matrix V = K[:, :D_V]: a key tile
// is fetched once into shared memory and serves as the B operand of both products (row-major for Q K^T, read
// transposed by ldmatrix for P V).  The causal mask follows the row's token: row r sees keys up to
// context - tokens + r / H.
//
// Two kernels.  latent_attention_mma_kernel, for steps with prompt portions: a block owns 16 * ROWW query rows of one
// request (ROWW = 4 in use) and walks all their keys.  Each group of 16 rows has VS warps that share the rows and split
// the D_V value columns between them (each computes the scores of the whole key tile itself; VS = 2 only with D_V = 512,
// where one warp's share of the output, 16 x 512 float32, would not fit its registers).  Key tiles of 32 rows go
// through NBUF buffers filled by cp.async, NBUF - 1 tiles on their way while one is multiplied (two in use: blocks of
// 64 rows leave room for no more when rows are long).  latent_decode_mma_kernel, for steps of single tokens (H rows per
// request: one tile of 16 for up to 16 heads): described where it stands; the keys are cut into `splits` ranges over
// blockIdx.z whose partial results (float32, with the base-2 logarithm of their sums) the shared merge kernel adds.
// In both, shared-memory rows are D_K + 8 elements apart, which puts the eight rows of an ldmatrix into eight different
// bank groups for every D_K that is a multiple of 16, and a key row's page is looked up once per tile at most.
#include "common.cuh"
#include "mma_common.cuh"

namespace ms {

constexpr int LBN = 32;       // keys per tile

template <int DV, int VS, int ROWW, int NBUF>
__global__ void __launch_bounds__(32 * VS * ROWW)
latent_attention_mma_kernel(const __nv_bfloat16* __restrict__ q_full, const __nv_bfloat16* __restrict__ cache,
                            const int* __restrict__ block_tables, int table_stride, const int* __restrict__ query_start,
                            const int* __restrict__ context_lens, int page_size, int heads, int dk, float scale_log2,
                            int window, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                            float* __restrict__ part_lse, int splits) {
  constexpr int DVW = DV / VS;          // value columns of one warp
  constexpr int THREADS = 32 * VS * ROWW;
  static_assert(DVW % 16 == 0, "a warp's share of the values must be a multiple of 16 columns");
  extern __shared__ __align__(16) unsigned char latent_smem[];
  grid_dependency_wait();
  grid_dependency_launch();
  const int dkp = dk + 8;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(latent_smem);     // [16 * ROWW][dkp]
  __nv_bfloat16* k_s = q_s + 16 * ROWW * dkp;                             // [NBUF][LBN][dkp]
  const int req = blockIdx.y, split = blockIdx.z;
  const int q0 = query_start[req], q_len = query_start[req + 1] - q0, ctx = context_lens[req];
  const int rows = q_len * heads;
  const int m0 = blockIdx.x * 16 * ROWW;
  if (m0 >= rows) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wr = warp / VS, wv = warp % VS;
  const int* table = block_tables + (size_t)req * table_stride;

  // the keys this block walks: up to the position of its last row, from the window's start of its first
  const int last_row = min(m0 + 16 * ROWW, rows) - 1;
  const int pos_last = ctx - q_len + last_row / heads;
  const int pos_first = ctx - q_len + m0 / heads;
  const int key_begin = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
  const int tile_begin = key_begin / LBN, tile_end = pos_last / LBN + 1;
  const int per_split = (tile_end - tile_begin + splits - 1) / splits;
  const int t_begin = tile_begin + split * per_split;
  const int t_end = min(tile_end, t_begin + per_split);

  const int chunks = dk >> 3;           // 16-byte pieces per row
  // A key row of a tile belongs to THREADS / 32 threads, which look its page up once and then request its pieces one
  // after the other (a lookup per piece would put a trip to the L2 cache before every request).
  constexpr int TPR = THREADS / LBN;
  static_assert(THREADS % LBN == 0 && TPR >= 1, "whole threads per key row");
  const int load_r = tid / TPR, load_c = tid % TPR;
  auto load_keys = [&](int tile, int buffer) {
    const int key = tile * LBN + load_r;
    const bool valid = key <= pos_last;
    const int page = valid ? table[key / page_size] : 0;
    const __nv_bfloat16* src = cache + ((size_t)page * page_size + (valid ? key % page_size : 0)) * dk;
    __nv_bfloat16* dst = k_s + ((size_t)buffer * LBN + load_r) * dkp;
    for (int c = load_c; c < chunks; c += TPR) cp_async_16(dst + c * 8, src + c * 8, valid);
  };
  if (t_begin < t_end) {
    const __nv_bfloat16* q_rows = q_full + ((size_t)q0 * heads + m0) * dk;
    for (int i = tid; i < 16 * ROWW * chunks; i += THREADS) {
      const int r = i / chunks, c = i % chunks;
      cp_async_16(q_s + r * dkp + c * 8, q_rows + (size_t)r * dk + c * 8, m0 + r < rows);
    }
    load_keys(t_begin, 0);
  }
  cp_async_commit();
#pragma unroll
  for (int ahead = 1; ahead < NBUF - 1; ++ahead) {
    if (t_begin + ahead < t_end) load_keys(t_begin + ahead, ahead);
    cp_async_commit();
  }

  // this thread's two rows of the 16: lane / 4 and lane / 4 + 8
  const int row_a = m0 + wr * 16 + (lane >> 2), row_b = row_a + 8;
  const int pos_a = row_a < rows ? ctx - q_len + row_a / heads : -1;     // -1: no key is visible (a row beyond the request's)
  const int pos_b = row_b < rows ? ctx - q_len + row_b / heads : -1;
  const int low_a = window > 0 ? pos_a - window : -2147483647, low_b = window > 0 ? pos_b - window : -2147483647;
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o[DVW / 8][4];
#pragma unroll
  for (int i = 0; i < DVW / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int tile = t_begin; tile < t_end; ++tile) {
    const int buffer = (tile - t_begin) % NBUF;
    cp_async_wait<NBUF - 2>();
    __syncthreads();      // this tile has arrived for everyone, and everyone is done with the tile before it,
    if (tile + NBUF - 1 < t_end) load_keys(tile + NBUF - 1, (tile - t_begin + NBUF - 1) % NBUF);      // whose buffer is refilled
    cp_async_commit();
    const __nv_bfloat16* kt = k_s + (size_t)buffer * LBN * dkp;

    float s[LBN / 8][4];
#pragma unroll
    for (int i = 0; i < LBN / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 2
    for (int kc = 0; kc < (dk >> 4); ++kc) {
      unsigned a[4];
      ldmatrix_x4(a, q_s + (wr * 16 + (lane & 15)) * dkp + kc * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int np = 0; np < LBN / 16; ++np) {
        unsigned b[4];
        ldmatrix_x4(b, kt + (np * 16 + (lane & 7) + (lane >> 4) * 8) * dkp + kc * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[2 * np], a, b[0], b[1]);
        mma_bf16(s[2 * np + 1], a, b[2], b[3]);
      }
    }
    // mask, running maximum and sum (base 2)
    float max_a = -INFINITY, max_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < LBN / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = tile * LBN + nt * 8 + (lane & 3) * 2 + e;
        s[nt][e] = (key <= pos_a && key > low_a) ? s[nt][e] * scale_log2 : -INFINITY;
        s[nt][2 + e] = (key <= pos_b && key > low_b) ? s[nt][2 + e] * scale_log2 : -INFINITY;
        max_a = fmaxf(max_a, s[nt][e]);
        max_b = fmaxf(max_b, s[nt][2 + e]);
      }
    }
    max_a = fmaxf(max_a, __shfl_xor_sync(0xffffffffu, max_a, 1));
    max_a = fmaxf(max_a, __shfl_xor_sync(0xffffffffu, max_a, 2));
    max_b = fmaxf(max_b, __shfl_xor_sync(0xffffffffu, max_b, 1));
    max_b = fmaxf(max_b, __shfl_xor_sync(0xffffffffu, max_b, 2));
    const float new_a = fmaxf(m_a, max_a), new_b = fmaxf(m_b, max_b);
    const float use_a = new_a == -INFINITY ? 0.f : new_a, use_b = new_b == -INFINITY ? 0.f : new_b;   // (nothing seen yet: all p are 0)
    const float corr_a = exp2f(m_a - use_a), corr_b = exp2f(m_b - use_b);
    m_a = new_a;
    m_b = new_b;
    float sum_a = 0.f, sum_b = 0.f;
    unsigned p[LBN / 16][4];
#pragma unroll
    for (int nt = 0; nt < LBN / 8; ++nt) {
      const float p0 = exp2f(s[nt][0] - use_a), p1 = exp2f(s[nt][1] - use_a);
      const float p2 = exp2f(s[nt][2] - use_b), p3 = exp2f(s[nt][3] - use_b);
      sum_a += p0 + p1;
      sum_b += p2 + p3;
      p[nt >> 1][(nt & 1) * 2] = pack_bf16(p0, p1);
      p[nt >> 1][(nt & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
    l_a = l_a * corr_a + sum_a;
    l_b = l_b * corr_b + sum_b;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) {
      o[i][0] *= corr_a;
      o[i][1] *= corr_a;
      o[i][2] *= corr_b;
      o[i][3] *= corr_b;
    }
    // O += P V with V the first D_V columns of the same tile, read transposed
#pragma unroll
    for (int kk = 0; kk < LBN / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < DVW / 16; ++np) {
        unsigned b[4];
        ldmatrix_x4_trans(b, kt + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * dkp + wv * DVW + np * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * np], p[kk], b[0], b[1]);
        mma_bf16(o[2 * np + 1], p[kk], b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  const size_t item_a = (size_t)q0 * heads + row_a, item_b = (size_t)q0 * heads + row_b;
  const int col0 = wv * DVW + (lane & 3) * 2;
  if (splits == 1) {
    const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) {
      if (row_a < rows)
        *reinterpret_cast<__nv_bfloat162*>(out + item_a * DV + col0 + i * 8) = __floats2bfloat162_rn(o[i][0] * inv_a, o[i][1] * inv_a);
      if (row_b < rows)
        *reinterpret_cast<__nv_bfloat162*>(out + item_b * DV + col0 + i * 8) = __floats2bfloat162_rn(o[i][2] * inv_b, o[i][3] * inv_b);
    }
    return;
  }
  // partial result of this split: its own softmax-weighted mean, and log2 of its sum of 2^score
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
  if (row_a < rows) {
    float* dst = part_o + (item_a * splits + split) * DV + col0;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][0] * inv_a, o[i][1] * inv_a);
    if (wv == 0 && (lane & 3) == 0) part_lse[item_a * splits + split] = l_a > 0.f ? m_a + log2f(l_a) : -INFINITY;
  }
  if (row_b < rows) {
    float* dst = part_o + (item_b * splits + split) * DV + col0;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2] * inv_b, o[i][3] * inv_b);
    if (wv == 0 && (lane & 3) == 0) part_lse[item_b * splits + split] = l_b > 0.f ? m_b + log2f(l_b) : -INFINITY;
  }
}

// Steps of single tokens: a request brings only H query rows (one tile of 16 for up to 16 heads), so a key tile cannot be
// shared by many row groups.  Instead the KW warps of a block share ONE key tile in another way: for the scores each
// takes LBN / KW of the tile's keys (all of D_K), masks them and finds its rows' maxima; the maxima meet in shared
// memory, every warp turns its own scores into probabilities with the common maximum and leaves them, as bfloat16,
// in shared memory, from where all warps fetch the whole tile's probabilities as A fragments; for P V each warp
// takes a KW-th of the value columns.  Nothing is computed twice, per tile a warp handles 16 x 8 scores instead of 16 x 32,
// and only 16 maxima and 1 KB of probabilities are exchanged.  Each warp keeps the sum of its own keys' probabilities
// (all relative to the same running maximum); the sums meet once, at the end.  Keys are cut into ranges over blockIdx.z
// as above, with NBUF key buffers; the block's part of the page table is fetched once.
constexpr int kDecodePages = 512;

template <int DV, int KW, int NBUF>
__global__ void __launch_bounds__(32 * KW)
latent_decode_mma_kernel(const __nv_bfloat16* __restrict__ q_full, const __nv_bfloat16* __restrict__ cache,
                         const int* __restrict__ block_tables, int table_stride, const int* __restrict__ query_start,
                         const int* __restrict__ context_lens, int page_size, int heads, int dk, float scale_log2,
                         int window, __nv_bfloat16* __restrict__ out, float* __restrict__ part_o,
                         float* __restrict__ part_lse, int splits) {
  constexpr int DVW = DV / KW;          // value columns of one warp
  constexpr int THREADS = 32 * KW;
  constexpr int NT = LBN / 8 / KW;      // tiles of 8 keys whose scores one warp computes
  constexpr int PLD = LBN + 8;          // elements between the rows of the exchanged probabilities
  static_assert(NT >= 1 && NT * 8 * KW == LBN, "the warps split the keys of a tile evenly");
  static_assert(DVW % 16 == 0, "a warp's share of the values must be a multiple of 16 columns");
  extern __shared__ __align__(16) unsigned char latent_smem[];
  grid_dependency_wait();
  grid_dependency_launch();
  const int dkp = dk + 8;
  __nv_bfloat16* q_s = reinterpret_cast<__nv_bfloat16*>(latent_smem);     // [16][dkp]
  __nv_bfloat16* k_s = q_s + 16 * dkp;                                    // [NBUF][LBN][dkp]
  __nv_bfloat16* p_x = k_s + (size_t)NBUF * LBN * dkp;                    // [16][PLD]: the tile's probabilities
  float* max_x = reinterpret_cast<float*>(p_x + 16 * PLD);                // [KW][16]: the warps' row maxima (at the end: sums)
  int* pages_s = reinterpret_cast<int*>(max_x + KW * 16);                 // [kDecodePages]: the block's part of the page table
  const int req = blockIdx.y, split = blockIdx.z;
  const int q0 = query_start[req], q_len = query_start[req + 1] - q0, ctx = context_lens[req];
  const int rows = q_len * heads;
  const int m0 = blockIdx.x * 16;
  if (m0 >= rows) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* table = block_tables + (size_t)req * table_stride;

  const int last_row = min(m0 + 16, rows) - 1;
  const int pos_last = ctx - q_len + last_row / heads;
  const int pos_first = ctx - q_len + m0 / heads;
  const int key_begin = (window > 0 && pos_first - window + 1 > 0) ? pos_first - window + 1 : 0;
  const int tile_begin = key_begin / LBN, tile_end = pos_last / LBN + 1;
  const int per_split = (tile_end - tile_begin + splits - 1) / splits;
  const int t_begin = tile_begin + split * per_split;
  const int t_end = min(tile_end, t_begin + per_split);

  // The pages of this block's keys, fetched once: a lookup in global memory before every tile's requests would put two
  // trips to memory, one after the other, into every tile (pages beyond the array's size are looked up as they come).
  const int first_page = t_begin < t_end ? (t_begin * LBN) / page_size : 0;
  const int n_pages = t_begin < t_end ? min(pos_last, t_end * LBN - 1) / page_size - first_page + 1 : 0;
  for (int i = tid; i < min(n_pages, kDecodePages); i += THREADS) pages_s[i] = table[first_page + i];
  __syncthreads();
  const int chunks = dk >> 3;
  constexpr int TPR = THREADS / LBN;
  static_assert(THREADS % LBN == 0 && TPR >= 1, "whole threads per key row");
  const int load_r = tid / TPR, load_c = tid % TPR;
  auto load_keys = [&](int tile, int buffer) {
    const int key = tile * LBN + load_r;
    const bool valid = key <= pos_last;
    const int page_index = key / page_size - first_page;
    const int page = !valid ? 0 : (page_index < kDecodePages ? pages_s[page_index] : table[first_page + page_index]);
    const __nv_bfloat16* src = cache + ((size_t)page * page_size + (valid ? key % page_size : 0)) * dk;
    __nv_bfloat16* dst = k_s + ((size_t)buffer * LBN + load_r) * dkp;
    for (int c = load_c; c < chunks; c += TPR) cp_async_16(dst + c * 8, src + c * 8, valid);
  };
  if (t_begin < t_end) {
    const __nv_bfloat16* q_rows = q_full + ((size_t)q0 * heads + m0) * dk;
    for (int i = tid; i < 16 * chunks; i += THREADS) {
      const int r = i / chunks, c = i % chunks;
      cp_async_16(q_s + r * dkp + c * 8, q_rows + (size_t)r * dk + c * 8, m0 + r < rows);
    }
    load_keys(t_begin, 0);
  }
  cp_async_commit();
#pragma unroll
  for (int ahead = 1; ahead < NBUF - 1; ++ahead) {
    if (t_begin + ahead < t_end) load_keys(t_begin + ahead, ahead);
    cp_async_commit();
  }

  const int row_a = m0 + (lane >> 2), row_b = row_a + 8;
  const int pos_a = row_a < rows ? ctx - q_len + row_a / heads : -1;
  const int pos_b = row_b < rows ? ctx - q_len + row_b / heads : -1;
  const int low_a = window > 0 ? pos_a - window : -2147483647, low_b = window > 0 ? pos_b - window : -2147483647;
  const int n_kc = dk >> 4;
  const int my_key0 = warp * NT * 8;     // this warp's keys of a tile
  float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
  float o[DVW / 8][4];
#pragma unroll
  for (int i = 0; i < DVW / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;

  for (int tile = t_begin; tile < t_end; ++tile) {
    const int buffer = (tile - t_begin) % NBUF;
    cp_async_wait<NBUF - 2>();
    __syncthreads();      // the tile is there for everyone; everyone has read the exchanged scores of the tile before
    if (tile + NBUF - 1 < t_end) load_keys(tile + NBUF - 1, (tile - t_begin + NBUF - 1) % NBUF);
    cp_async_commit();
    const __nv_bfloat16* kt = k_s + (size_t)buffer * LBN * dkp;

    // scores of this warp's keys: two chains of products (even and odd steps of 16 along the row) added at the end
    float s[NT][4], s_odd[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = s_odd[i][0] = s_odd[i][1] = s_odd[i][2] = s_odd[i][3] = 0.f;
    for (int kc = 0; kc + 1 < n_kc; kc += 2) {
      unsigned a0[4], a1[4];
      ldmatrix_x4(a0, q_s + (lane & 15) * dkp + kc * 16 + (lane >> 4) * 8);
      ldmatrix_x4(a1, q_s + (lane & 15) * dkp + (kc + 1) * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        unsigned b[4];      // eight keys x 32 numbers of their rows: the B fragments of two steps
        ldmatrix_x4(b, kt + (my_key0 + nt * 8 + (lane & 7)) * dkp + kc * 16 + (lane >> 3) * 8);
        mma_bf16(s[nt], a0, b[0], b[1]);
        mma_bf16(s_odd[nt], a1, b[2], b[3]);
      }
    }
    if (n_kc & 1) {
      const int kc = n_kc - 1;
      unsigned a0[4];
      ldmatrix_x4(a0, q_s + (lane & 15) * dkp + kc * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        unsigned b[4];      // (the upper sixteen lanes repeat the addresses of the lower: only b[0], b[1] are used)
        ldmatrix_x4(b, kt + (my_key0 + nt * 8 + (lane & 7)) * dkp + kc * 16 + ((lane >> 3) & 1) * 8);
        mma_bf16(s[nt], a0, b[0], b[1]);
      }
    }
    float max_a = -INFINITY, max_b = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int key = tile * LBN + my_key0 + nt * 8 + (lane & 3) * 2 + e;
        s[nt][e] = (key <= pos_a && key > low_a) ? (s[nt][e] + s_odd[nt][e]) * scale_log2 : -INFINITY;
        s[nt][2 + e] = (key <= pos_b && key > low_b) ? (s[nt][2 + e] + s_odd[nt][2 + e]) * scale_log2 : -INFINITY;
        max_a = fmaxf(max_a, s[nt][e]);
        max_b = fmaxf(max_b, s[nt][2 + e]);
      }
    }
    max_a = fmaxf(max_a, __shfl_xor_sync(0xffffffffu, max_a, 1));
    max_a = fmaxf(max_a, __shfl_xor_sync(0xffffffffu, max_a, 2));
    max_b = fmaxf(max_b, __shfl_xor_sync(0xffffffffu, max_b, 1));
    max_b = fmaxf(max_b, __shfl_xor_sync(0xffffffffu, max_b, 2));
    if ((lane & 3) == 0) {
      max_x[warp * 16 + (lane >> 2)] = max_a;
      max_x[warp * 16 + (lane >> 2) + 8] = max_b;
    }
    __syncthreads();
    float new_a = m_a, new_b = m_b;
#pragma unroll
    for (int w = 0; w < KW; ++w) {
      new_a = fmaxf(new_a, max_x[w * 16 + (lane >> 2)]);
      new_b = fmaxf(new_b, max_x[w * 16 + (lane >> 2) + 8]);
    }
    const float use_a = new_a == -INFINITY ? 0.f : new_a, use_b = new_b == -INFINITY ? 0.f : new_b;
    const float corr_a = exp2f(m_a - use_a), corr_b = exp2f(m_b - use_b);
    m_a = new_a;
    m_b = new_b;
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      const float p0 = exp2f(s[nt][0] - use_a), p1 = exp2f(s[nt][1] - use_a);
      const float p2 = exp2f(s[nt][2] - use_b), p3 = exp2f(s[nt][3] - use_b);
      sum_a += p0 + p1;
      sum_b += p2 + p3;
      const int col = my_key0 + nt * 8 + (lane & 3) * 2;
      *reinterpret_cast<__nv_bfloat162*>(p_x + (lane >> 2) * PLD + col) = __floats2bfloat162_rn(p0, p1);
      *reinterpret_cast<__nv_bfloat162*>(p_x + ((lane >> 2) + 8) * PLD + col) = __floats2bfloat162_rn(p2, p3);
    }
    l_a = l_a * corr_a + sum_a;       // (of this warp's keys only)
    l_b = l_b * corr_b + sum_b;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) {
      o[i][0] *= corr_a;
      o[i][1] *= corr_a;
      o[i][2] *= corr_b;
      o[i][3] *= corr_b;
    }
    __syncthreads();
    unsigned p[LBN / 16][4];
#pragma unroll
    for (int kk = 0; kk < LBN / 16; ++kk) ldmatrix_x4(p[kk], p_x + (lane & 15) * PLD + kk * 16 + (lane >> 4) * 8);
#pragma unroll
    for (int kk = 0; kk < LBN / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < DVW / 16; ++np) {
        unsigned b[4];
        ldmatrix_x4_trans(b, kt + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * dkp + warp * DVW + np * 16 + (lane >> 4) * 8);
        mma_bf16(o[2 * np], p[kk], b[0], b[1]);
        mma_bf16(o[2 * np + 1], p[kk], b[2], b[3]);
      }
    }
  }
  cp_async_wait<0>();

  l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
  l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
  l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
  // the warps' sums (each over its own keys, all relative to the same maximum) meet, added in warp order
  if ((lane & 3) == 0) {
    max_x[warp * 16 + (lane >> 2)] = l_a;
    max_x[warp * 16 + (lane >> 2) + 8] = l_b;
  }
  __syncthreads();
  l_a = l_b = 0.f;
#pragma unroll
  for (int w = 0; w < KW; ++w) {
    l_a += max_x[w * 16 + (lane >> 2)];
    l_b += max_x[w * 16 + (lane >> 2) + 8];
  }
  const size_t item_a = (size_t)q0 * heads + row_a, item_b = (size_t)q0 * heads + row_b;
  const int col0 = warp * DVW + (lane & 3) * 2;
  const float inv_a = l_a > 0.f ? 1.f / l_a : 0.f, inv_b = l_b > 0.f ? 1.f / l_b : 0.f;
  if (splits == 1) {
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) {
      if (row_a < rows)
        *reinterpret_cast<__nv_bfloat162*>(out + item_a * DV + col0 + i * 8) = __floats2bfloat162_rn(o[i][0] * inv_a, o[i][1] * inv_a);
      if (row_b < rows)
        *reinterpret_cast<__nv_bfloat162*>(out + item_b * DV + col0 + i * 8) = __floats2bfloat162_rn(o[i][2] * inv_b, o[i][3] * inv_b);
    }
    return;
  }
  if (row_a < rows) {
    float* dst = part_o + (item_a * splits + split) * DV + col0;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][0] * inv_a, o[i][1] * inv_a);
    if (warp == 0 && (lane & 3) == 0) part_lse[item_a * splits + split] = l_a > 0.f ? m_a + log2f(l_a) : -INFINITY;
  }
  if (row_b < rows) {
    float* dst = part_o + (item_b * splits + split) * DV + col0;
#pragma unroll
    for (int i = 0; i < DVW / 8; ++i) *reinterpret_cast<float2*>(dst + i * 8) = make_float2(o[i][2] * inv_b, o[i][3] * inv_b);
    if (warp == 0 && (lane & 3) == 0) part_lse[item_b * splits + split] = l_b > 0.f ? m_b + log2f(l_b) : -INFINITY;
  }
}

static int g_latent_sms = 0;

static int latent_sm_count() {
  if (g_latent_sms == 0) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&g_latent_sms, cudaDevAttrMultiProcessorCount, device);
    if (g_latent_sms <= 0) g_latent_sms = 148;
  }
  return g_latent_sms;
}

template <int DV, int VS, int ROWW, int NBUF>
static int launch_latent(const __nv_bfloat16* q_full, const __nv_bfloat16* cache, const int* block_tables, int table_stride,
                         const int* query_start, const int* context_lens, int page_size, int heads, int dk, float scale,
                         int window, __nv_bfloat16* out, float* part_o, float* part_lse, int splits, int n_requests,
                         int max_query_len, cudaStream_t stream) {
  const size_t smem = (size_t)(16 * ROWW + NBUF * LBN) * (dk + 8) * sizeof(__nv_bfloat16);
  static size_t allowed = 0;       // per instantiation
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(latent_attention_mma_kernel<DV, VS, ROWW, NBUF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem);
    if (e != cudaSuccess) MS_FAIL("latent_attention_mma: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    allowed = smem;
  }
  const long long rows = (long long)max_query_len * heads;
  dim3 grid((unsigned)((rows + 16 * ROWW - 1) / (16 * ROWW)), n_requests, splits);
  ms::launch(latent_attention_mma_kernel<DV, VS, ROWW, NBUF>, grid, 32 * VS * ROWW, smem, stream, q_full, cache, block_tables,
             table_stride, query_start, context_lens, page_size, heads, dk, scale * 1.4426950408889634f, window, out, part_o,
             part_lse, splits);
  MS_CHECK_LAUNCH("latent_attention_mma");
  return 0;
}

template <int DV, int KW, int NBUF>
static int launch_latent_decode(const __nv_bfloat16* q_full, const __nv_bfloat16* cache, const int* block_tables, int table_stride,
                                const int* query_start, const int* context_lens, int page_size, int heads, int dk, float scale,
                                int window, __nv_bfloat16* out, float* part_o, float* part_lse, int splits, int n_requests,
                                int max_query_len, cudaStream_t stream) {
  const size_t smem = (size_t)(16 + NBUF * LBN) * (dk + 8) * sizeof(__nv_bfloat16) + (size_t)16 * (LBN + 8) * sizeof(__nv_bfloat16)
                      + (size_t)KW * 16 * sizeof(float) + kDecodePages * sizeof(int);
  static size_t allowed = 0;       // per instantiation
  if (smem > allowed) {
    cudaError_t e = cudaFuncSetAttribute(latent_decode_mma_kernel<DV, KW, NBUF>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) MS_FAIL("latent_attention_mma: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    allowed = smem;
  }
  const long long rows = (long long)max_query_len * heads;
  dim3 grid((unsigned)((rows + 15) / 16), n_requests, splits);
  ms::launch(latent_decode_mma_kernel<DV, KW, NBUF>, grid, 32 * KW, smem, stream, q_full, cache, block_tables, table_stride,
             query_start, context_lens, page_size, heads, dk, scale * 1.4426950408889634f, window, out, part_o, part_lse, splits);
  MS_CHECK_LAUNCH("latent_attention_mma (single tokens)");
  return 0;
}

}  // namespace ms

using namespace ms;

// Sizes the tensor-core kernel takes: a latent of 64, 96, 128, 256 or 512 numbers, a rotated part that is a multiple
// of 16 (or empty), rows of at most 1024 numbers.
MS_EXPORT int ms_latent_attention_mma_supports(int rank, int rot, int heads) {
  const bool rank_ok = rank == 64 || rank == 96 || rank == 128 || rank == 256 || rank == 512;
  return rank_ok && rot >= 0 && rot % 16 == 0 && rank + rot <= 1024 && heads >= 1 && heads <= 65535 ? 1 : 0;
}

// How many ranges the keys of a step are cut into: 1 for steps with prompt portions; for steps of single tokens enough
// that the blocks fill the multiprocessors about four times, at most one range per two key tiles of the longest
// context (`max_context_len`, an upper bound), and at most 32 (16 for a latent of 512: the merge that takes more
// than 16 ranges holds sixteen partial results per thread).
MS_EXPORT int ms_latent_attention_mma_splits(int rank, int rot, int heads, int n_requests, int max_query_len,
                                             int max_context_len) {
  if (max_query_len != 1 || n_requests <= 0) return 1;
  const int row_tiles = (heads + 15) / 16;
  const int blocks = n_requests * row_tiles;
  int splits = (4 * latent_sm_count() + blocks - 1) / blocks;
  const int by_keys = (max_context_len + 2 * LBN - 1) / (2 * LBN);
  const int most = rank > 256 ? 16 : 32;
  if (splits > by_keys) splits = by_keys;
  if (splits > most) splits = most;
  return splits < 1 ? 1 : splits;
}

// q_full [n_tokens, heads, rank + rot] and out [n_tokens, heads, rank] bfloat16; cache [pages, page_size, rank + rot];
// part_o float32 [n_tokens * heads * splits, rank] and part_lse [n_tokens * heads * splits] when splits > 1.
MS_EXPORT int ms_latent_attention_mma(const void* q_full, const void* cache, const int* block_tables, int table_stride,
                                      const int* query_start, const int* context_lens, int page_size, int heads, int rank,
                                      int rot, float scale, int window, void* out, float* part_o, float* part_lse, int splits,
                                      int n_requests, int max_query_len, int n_tokens, cudaStream_t stream) {
  if (n_tokens == 0 || n_requests == 0) return 0;
  MS_REQUIRE(ms_latent_attention_mma_supports(rank, rot, heads), "latent_attention_mma: sizes %d + %d are not supported", rank, rot);
  MS_REQUIRE(page_size > 0 && max_query_len > 0, "latent_attention_mma: page size %d, longest portion %d", page_size, max_query_len);
  MS_REQUIRE(splits >= 1 && splits <= (rank > 256 ? 16 : 32) && (splits == 1 || (part_o && part_lse)), "latent_attention_mma: %d splits", splits);
  MS_REQUIRE(n_requests <= 65535, "latent_attention_mma: %d requests in one launch is too many", n_requests);
  const int dk = rank + rot;
  const bool single = max_query_len == 1;
  const __nv_bfloat16* q = (const __nv_bfloat16*)q_full;
  const __nv_bfloat16* c = (const __nv_bfloat16*)cache;
  __nv_bfloat16* o = (__nv_bfloat16*)out;
  int code = 0;
  // Steps of single tokens: the kernel whose warps share every key tile (KW warps; four key buffers).  Steps with prompt
  // portions: blocks of 64 rows, VS warps per row group (two for a latent of 512, whose output would not fit one warp's
  // registers; the two then compute every score twice).
#define MS_LATENT_CASE(DV, KW, VS)                                                                                                  \
  if (rank == DV) {                                                                                                                 \
    code = single ? launch_latent_decode<DV, KW, 4>(q, c, block_tables, table_stride, query_start, context_lens, page_size, heads,  \
                                                    dk, scale, window, o, part_o, part_lse, splits, n_requests, max_query_len, stream) \
                  : launch_latent<DV, VS, 4, 2>(q, c, block_tables, table_stride, query_start, context_lens, page_size, heads, dk,  \
                                                scale, window, o, part_o, part_lse, splits, n_requests, max_query_len, stream);     \
    if (code) return code;                                                                                                          \
  }
  MS_LATENT_CASE(64, 4, 1)
  MS_LATENT_CASE(96, 2, 1)
  MS_LATENT_CASE(128, 4, 1)
  MS_LATENT_CASE(256, 4, 1)
  MS_LATENT_CASE(512, 4, 2)
#undef MS_LATENT_CASE
  if (splits > 1) {
    const int items = n_tokens * heads;
    if (rank == 64) launch_attention_combine<64>(part_o, part_lse, o, splits, items, stream);
    else if (rank == 96) launch_attention_combine<96>(part_o, part_lse, o, splits, items, stream);
    else if (rank == 128) launch_attention_combine<128>(part_o, part_lse, o, splits, items, stream);
    else if (rank == 256) launch_attention_combine<256>(part_o, part_lse, o, splits, items, stream);
    else launch_attention_combine<512>(part_o, part_lse, o, splits, items, stream);
    MS_CHECK_LAUNCH("latent_attention_mma: merge of the key ranges");
  }
  return 0;
}
