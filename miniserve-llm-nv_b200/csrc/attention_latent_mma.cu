// Tensor-core form of the latent attention (placeholder while the kernel is brought up: it takes no sizes yet, so
// every call runs the general kernel).
#include "common.cuh"

MS_EXPORT int ms_latent_attention_mma_supports(int rank, int rot, int heads) { return 0; }

MS_EXPORT int ms_latent_attention_mma_splits(int rank, int rot, int heads, int n_requests, int max_query_len,
                                             int max_context_len) { return 1; }

MS_EXPORT int ms_latent_attention_mma(const void* q_full, const void* cache, const int* block_tables, int table_stride,
                                      const int* query_start, const int* context_lens, int page_size, int heads, int rank,
                                      int rot, float scale, int window, void* out, float* part_o, float* part_lse, int splits,
                                      int n_requests, int max_query_len, int n_tokens, cudaStream_t stream) {
  MS_FAIL("latent_attention_mma: no sizes are supported yet");
}
