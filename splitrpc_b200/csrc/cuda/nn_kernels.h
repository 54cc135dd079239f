// Launch API of the memory-bound layers (pooling, normalisation, softmax response
// writers, embedding, attention).  Pointers are device addresses; `d_stub` is the
// device-visible g_params stub of an app context (may be null when a direct
// pointer is given).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

cudaError_t nn_stem_im2col(const void* d_stub, const float* direct_in, int batch, void* out, const float mean[3],
                           const float inv_std[3], cudaStream_t s);
// Space-to-depth form of the same input: out[batch][115][115][16] bf16 (see nn_kernels.cu).
cudaError_t nn_stem_s2d(const void* d_stub, const float* direct_in, int batch, void* out, const float mean[3],
                        const float inv_std[3], cudaStream_t s);
cudaError_t nn_maxpool3x3s2(const void* in, void* out, int n, int h, int w, int c, cudaStream_t s);
cudaError_t nn_global_avgpool(const void* in, void* out, int n, int hw, int c, cudaStream_t s);
// out[M, N] (fp32) = a[M, K] . w[N, K]^T + bias for a few rows (SIMT, weights staged in shared memory): the shape where a
// 128-row tensor-core tile leaves most of the GPU idle.  K a multiple of 8 up to 6400; lda, ldw multiples of 8.
cudaError_t nn_fc_skinny(const void* a, int lda, const void* w, int ldw, const float* bias, float* out, int ldo, int M, int N, int K,
                         cudaStream_t s);
cudaError_t nn_softmax_response(const float* logits, int rows, int n, int ld, const void* d_stub, void* direct_out,
                                size_t resp_stride, int write_argmax, uint32_t* counter, uint32_t* flag, uint32_t flag_value,
                                cudaStream_t s, const void* d_push = nullptr);
cudaError_t nn_layernorm(const void* x, const void* residual, const float* gamma, const float* beta, void* y, int rows,
                         int hidden, float eps, cudaStream_t s);
cudaError_t nn_bert_embed_ln(const void* d_stub, const int* direct_ids, size_t req_stride, int batch, int seq, const void* word,
                             const void* pos, const void* type, const float* gamma, const float* beta, void* y, int hidden,
                             int vocab, float eps, cudaStream_t s);
// Tensor-core attention: qk = [tokens, 2*hidden] (Q | K), vt = [hidden, tokens] (V transposed), out = [tokens, hidden].
cudaError_t nn_attention_tc(const void* qk, int ld_qk, const void* vt, int ld_vt, void* out, int ld_out, const float* v_bias,
                            int batch, int seq, int heads, uint32_t* status, cudaStream_t s);
cudaError_t nn_attention_d64(const void* qkv, void* out, int batch, int seq, int heads, int ld_qkv, int q_off, int k_off,
                             int v_off, int ld_out, cudaStream_t s);
