// Host launch API of hybrid.cu (recurrent mixers, latent attention with a sink, output-side norms).  `f32` selects the activation
// type of the call: float (exact mode) or bf16 (serving); norm weights, recurrence constants and states are always float.
#pragma once
#include <cuda_runtime.h>

namespace b200 {
cudaError_t gather_rows_launch(const void* table, bool table_f32, long long ld, const long long* ids, int col0, int n, void* out,
                               bool out_f32, int T, cudaStream_t s);
cudaError_t side_gate_launch(const void* gx, long long ld_g, const void* table, long long ld_t, const long long* ids, int col0, int n,
                             void* out, bool f32, int T, cudaStream_t s);
cudaError_t gelu_erf_launch(void* x, long long ld, int n, bool f32, int T, cudaStream_t s);
cudaError_t post_norm_add_launch(float* x, const float* y, long long ld_y, const float* w, void* xa, bool f32, int n, float eps, int T,
                                 cudaStream_t s);
cudaError_t rmsnorm_cast_launch(const float* x, long long ld_x, const float* w, void* out, bool f32, int n, float eps, int T, cudaStream_t s);
cudaError_t gated_rmsnorm_launch(const float* y, const void* g, long long ld_g, const float* w, void* out, bool f32, int C, int groups,
                                 int mode, float eps, int T, cudaStream_t s);
cudaError_t causal_conv_silu_launch(const void* u, long long ld_u, const float* w, const float* bias, void* cstate, const int* cu,
                                    const int* ctx, const int* slots, int B, int C, int K, void* out, bool f32, int T, cudaStream_t s);
cudaError_t ssm_scan_launch(const void* xbc, long long ld_x, const void* dt, long long ld_dt, const float* dt_bias, const float* A_log,
                            const float* D, float* state, const int* cu, const int* ctx, const int* slots, float* out, int B, int H, int N,
                            int P, int G, bool f32, int max_q, cudaStream_t s);
cudaError_t decay_scan_launch(const void* qkv, long long ld, const float* decay, float* state, const int* cu, const int* ctx,
                              const int* slots, float* out, int B, int H, int N, int P, bool f32, int max_q, cudaStream_t s);
cudaError_t latent_prologue_launch(const void* x, long long ld_x, int Qr, int L, int R, const float* qn_w, const float* kvn_w, float eps,
                                   void* cq, void* pool, const int* slot_map, const int* positions, const float* inv_freq, bool f32, int T,
                                   int interleaved, cudaStream_t s);
cudaError_t latent_attention_launch(const void* q, const void* pool, const float* sink, const int* block_tables, int max_blocks,
                                    const int* positions, const int* cu, int B, int H, int L, int R, int page, float scale,
                                    const float* inv_freq, void* out, bool f32, int T, int nsplit, int chunk, float* part, int window,
                                    int interleaved, cudaStream_t s);
cudaError_t rotate_half_launch(void* q, const int* positions, const float* inv_freq, int H, int L, int R, bool f32, int T, int interleaved,
                               cudaStream_t s);
cudaError_t sink_softmax_launch(const float* sc, const float* sink, int H, int n, int ctx0, float scale, void* out, bool f32, long long rows,
                                int window, int k0, float softcap, float temp_coef, float temp_every, cudaStream_t s);
// pre-norm residual step, mLSTM scan, sigmoid router, clamped-GLU experts (sink / ls / extra / row_of / scale may be nullptr)
cudaError_t scaled_add_norm_launch(float* x, const float* y, long long ld_y, const float* ls, const float* extra, long long ld_e,
                                   const float* gate, long long ld_gate, const float* w, void* xa, bool f32, int n, float eps, int T,
                                   cudaStream_t s);
cudaError_t mlstm_scan_launch(const void* in, long long ld_in, const float* gates, long long ld_g, const float* gate_bias, float* S, float* n,
                              float* m, const int* cu, const int* ctx, const int* slots, float* out, int B, int H, int N, int P, int PB,
                              float cap, float q_scale, bool f32, int max_q, cudaStream_t s);
// mode 0: sigmoid scores, weights = chosen scores; mode 1: logits + bias, weights = softmax over the chosen logits
cudaError_t router_topk_launch(const float* z, long long ld_z, const float* bias, int mode, int E, int top, int* idx, float* w, int T,
                               cudaStream_t s);
// kind 0: clamped GLU (limit); kind 1: silu(g) * u * scale
cudaError_t clamped_glu_launch(const void* g, long long ld_g, const void* u, long long ld_u, int F, float limit, const int* row_of,
                               const float* scale, void* out, bool f32, int rows, int kind, cudaStream_t s);
cudaError_t expert_rows_linear_launch(const void* x, long long ld_x, int div, const void* W, const int* expert, int N, int K, void* out, bool f32,
                                      bool out_f32, int rows, cudaStream_t s);
cudaError_t gather_sum_launch(const float* y, const int* row_of, const float* wts, int k, int n, float* out, int T, cudaStream_t s);
}  // namespace b200
