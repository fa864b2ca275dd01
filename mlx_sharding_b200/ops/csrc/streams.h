// Host launch API of streams.cu (several residual streams with dynamic-tanh norms, gated delta rule, attention with a sink inside
// blocks of positions, minGRU, group-limited softmax router).  `f32` selects the activation type of the call: float (exact mode) or
// bf16 (serving); streams, norm weights, recurrence constants and states are always float.  Nullable pointers are marked.
#pragma once
#include <cuda_runtime.h>

namespace b200 {
cudaError_t stream_embed_launch(const void* table, bool table_f32, long long ld, const long long* ids, float scale, int S, int n, float* xs, int T,
                                cudaStream_t s);
// y == nullptr: only the read.  y2, gate, ls nullable.
cudaError_t hyper_step_launch(float* xs, const float* y, long long ld_y, const float* y2, long long ld_y2, const void* gate, long long ld_g,
                              const float* ls, const float* mix, const float* out_w, float mult, const float* in_w, float alpha, const float* w,
                              const float* b, void* xa, bool f32, int S, int n, int T, cudaStream_t s);
cudaError_t relu2_launch(void* x, long long ld, int n, bool f32, int T, cudaStream_t s);
cudaError_t delta_scan_launch(const void* in, long long ld_in, const void* beta, long long ld_b, const float* dt, long long ld_dt,
                              const float* dt_bias, const float* A_log, float* state, const int* cu, const int* ctx, const int* slots, float* out,
                              int B, int H, int G, int N, int P, float q_scale, float unit_eps, bool f32, int max_q, float* pre, int T, cudaStream_t s);
// true: the step runs the register form of the scan, which takes a workspace `pre` of T * delta_scan_prepare_width(..) floats (token-wise
// operands, computed once per step)
bool delta_scan_wants_prepare(int N, int max_q);
long long delta_scan_prepare_width(int G, int H, int N, int P);
cudaError_t mingru_scan_launch(const void* rows, long long ld, int z0, int x0, int g0, int R, float* state, const int* cu, const int* ctx,
                               const int* slots, float out_mult, void* out, long long ld_out, int B, bool f32, int max_q, cudaStream_t s);
cudaError_t qk_norm_rope_append_launch(const void* rows, long long ld, int q0, int k0, int v0, int H, int G, int D, int V, const float* qn,
                                       const float* kn, float eps, const float* inv_freq, int rot, const int* positions, const int* slot_map,
                                       int page, float* qout, void* kpool, void* vpool, bool f32, int T, cudaStream_t s);
int sink_attention_warps(int H, int G);
// sink nullable; block / window 0 = no such limit; part: [T, H, nsplit, V + 2] floats when nsplit > 1
cudaError_t sink_attention_launch(const float* q, const void* kpool, const void* vpool, const float* sink, const int* block_tables, int max_blocks,
                                  const int* positions, const int* cu, int B, int H, int G, int D, int V, int page, int block, int window,
                                  float scale, float out_mult, void* out, long long ld_out, bool f32, int T, int nsplit, int chunk, float* part,
                                  cudaStream_t s);
cudaError_t group_softmax_topk_launch(const float* z, long long ld_z, const float* corr, int E, int top, int ng, int keep, int* idx, float* w, int T,
                                      cudaStream_t s);
}  // namespace b200
