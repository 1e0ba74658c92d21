// Launchers of the non-GEMM kernels (elementwise.cu, attn_*.cu, compress.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fc {

constexpr int DECODE_MAX_SPLITS = 32;

void launch_rms_norm(const void* x, void* residual, const void* w, void* y, long long T, int H, float eps,
                     cudaStream_t s);
void launch_layer_norm(const void* x, const void* w, const void* b, void* y, long long T, int H, float eps,
                       cudaStream_t s);
void launch_silu_and_mul(const void* x, void* y, long long T, int I, cudaStream_t s);
void launch_embedding(const void* ids, const void* weight, void* out, int T, int H, int V, int vocab_start,
                      cudaStream_t s);
void launch_rope_qknorm_store(const void* qkv, const void* positions, const void* cos_sin, const void* q_w,
                              const void* k_w, void* q_out, void* k_cache, void* v_cache, const void* slots, int T,
                              int Hq, int Hkv, int D, float eps, long long num_slots, int block_size,
                              uint32_t* status, cudaStream_t s, const float* partial = nullptr, int splits = 0,
                              long long split_stride = 0);   // partial != nullptr (head_dim 128 only): qkv is still
                                                             // fp32 split-K partial sums [splits, T, heads * D]
// out: int64 [B + 1] when `status` is given (the last entry receives the status code), else [B].  Column j of
// the logits is vocabulary entry vocab_offset + j; entries >= v_limit (-1: none) are padding.
void launch_sample(const void* logits, const void* temps, void* out, int B, int V, long long ld, uint32_t seed,
                   cudaStream_t s, int vocab_offset = 0, int v_limit = -1, const uint32_t* status = nullptr);

int decode_attn_pick_splits(int B, int Hkv, int max_ctx, int num_sms);
void launch_decode_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                             const int* context_lens, void* out, float* part_o, float* part_lse, int B, int Hq,
                             int Hkv, int D, int block_size, int max_blocks, int num_blocks, int splits,
                             float scale, uint32_t* status, cudaStream_t stream, int* merge_counters = nullptr);
void launch_prefill_attention(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                              const int* cu_seqlens_q, const int* kv_lens, void* out, int num_seqs, int max_q_len,
                              int Hq, int Hkv, int D, int block_size, int max_blocks, int num_blocks, float scale,
                              uint32_t* status, cudaStream_t stream);
// tcgen05 version (head_dim 128, block_size a multiple of 8)
bool prefill_attention_tc_supported(int D, int block_size);
void launch_prefill_attention_tc(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                 const int* cu_seqlens_q, const int* kv_lens, void* out, long long total_q,
                                 int num_seqs, int max_q_len, int Hq, int Hkv, int block_size, int max_blocks,
                                 int num_blocks, float scale, uint32_t* status, cudaStream_t stream);
// two query tiles per CTA in ping-pong, P and O in tensor memory (same limits)
void launch_prefill_attention_tc2(const void* q, const void* k_cache, const void* v_cache, const int* block_tables,
                                  const int* cu_seqlens_q, const int* kv_lens, void* out, long long total_q,
                                  int num_seqs, int max_q_len, int Hq, int Hkv, int block_size, int max_blocks,
                                  int num_blocks, float scale, uint32_t* status, cudaStream_t stream);
}  // namespace fc

namespace fc {
void launch_knorm_scores(const void* pool, const int* block_tables, const int* kv_lens, float* scores, int n_seq,
                         int L, int num_blocks, int block_size, int Hkv, int D, int max_blocks, int max_len,
                         int s_stride, int mode, uint32_t* status, cudaStream_t stream);
void launch_snapkv_scores(const void* pool, const void* qw, const int* block_tables, const int* kv_lens, float* votes,
                          float* scores, int n_seq, int L, int num_blocks, int Hkv, int Hq, int block_size, int D,
                          int max_blocks, int stride, int w, int kernel_size, float scale, uint32_t* status,
                          cudaStream_t stream);
void launch_expected_attention_scores(const void* pool, const void* qw, const int* block_tables, const int* kv_lens,
                                      float* stats, float* scores, int n_seq, int L, int num_blocks, int Hkv, int Hq,
                                      int block_size, int D, int max_blocks, int stride, int w, int n_sink,
                                      uint32_t* status, cudaStream_t stream, void* sig16 = nullptr);
// tcgen05 form of the SnapKV votes (head_dim 128, (Hq / Hkv) * window a multiple of 64): on unless FC_SNAPKV_TC=0
bool snapkv_tensor_cores();
void set_snapkv_tensor_cores(bool on);
// tcgen05 form of the ExpectedAttention scores (head_dim 128, needs the `sig16` scratch): on unless FC_EA_TC=0
bool ea_tensor_cores();
void set_ea_tensor_cores(bool on);
void launch_position_scores(float* scores, const int* kv_lens, int n_seq, int units_per_seq, int stride, int n_sink,
                            cudaStream_t stream);
void launch_select_compact(void* pool, const float* scores, const int* block_tables, const int* kv_lens,
                           const int* n_kepts, int n_seq, int L, int num_blocks, int block_size, int Hkv, int D,
                           int max_blocks, int s_stride, uint32_t* status, cudaStream_t stream);
}  // namespace fc

namespace fc {
void launch_dense_attention(const void* q, const void* k, const void* v, void* out, const uint8_t* key_mask,
                            int B, int Sq, int Sk, int H, int D, const long long* q_strides,
                            const long long* k_strides, const long long* v_strides, float scale,
                            cudaStream_t stream);
// The same on tcgen05 (attn_dense_tc.cu).  key_mask rows are padded with zeros to mask_ld bytes, a multiple of 128.
bool dense_attention_tc_supported(int B, int Sq, int Sk, int H, int D, const long long* q_strides,
                                  const long long* k_strides, const long long* v_strides);
void launch_dense_attention_tc(const void* q, const void* k, const void* v, void* out, const uint8_t* key_mask,
                               int mask_ld, int B, int Sq, int Sk, int H, int D, const long long* q_strides,
                               const long long* k_strides, const long long* v_strides, float scale,
                               uint32_t* status, cudaStream_t stream);
}  // namespace fc

namespace fc {
void launch_ccm_fused(void* pool, const int* block_tables, const int* kv_lens, const int* image_lens,
                      const void* w1, const void* w2, const void* w3, const void* b1, const void* b2,
                      const void* b3, int n_seq, int n_weight_layers, int layer_start, int layer_end,
                      int weight_layer_start, int num_blocks, int Hkv, int block_size, int D, int max_blocks,
                      int factor, int min_seq_len, int single_segment, int heads_per_cta, uint32_t* status,
                      cudaStream_t stream, const int* dst_block_tables = nullptr);
// dst_block_tables [n_seq, max_blocks]: write the compressed rows into these blocks instead of the leading rows
// of the request's own blocks (which then stay as they are).

// consumers of split-K partial sums [splits, T, N] fp32 (partials.cu)
void launch_add_rms_norm_partials(const float* partial, int splits, long long split_stride, const void* bias,
                                  void* residual, const void* w, void* y, long long T, int H, float eps,
                                  cudaStream_t s);
void launch_silu_mul_partials(const float* partial, int splits, long long split_stride, void* out, long long T,
                              int I, cudaStream_t s);
}  // namespace fc

namespace fc {
// KV quantisers (quant.cu).  x: bf16 [groups, g]; codes: one byte per value (INT8, FP8) or per two values (INT4,
// NF4: even index in the low nibble); scale [groups] fp32 (the absmax for the 4-bit modes); zero [groups] for
// the asymmetric mode.  y_fake != nullptr: write decode(encode(x)) there instead of codes and scales.
enum QuantMode : int { QUANT_INT8 = 0, QUANT_INT8_ASYM = 1, QUANT_INT4 = 2, QUANT_NF4 = 3, QUANT_FP8_E4M3 = 4,
                       QUANT_FP8_E5M2 = 5 };
void launch_quantize(const void* x, void* q, float* scale, float* zero, void* y_fake, long long groups, int g,
                     int mode, cudaStream_t s);
void launch_dequantize(const void* q, const float* scale, const float* zero, void* y, long long groups, int g,
                       int mode, cudaStream_t s);
}  // namespace fc
