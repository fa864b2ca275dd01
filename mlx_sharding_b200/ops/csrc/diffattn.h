// Host launch API of diffattn.cu (layer norms on the fp32 residual stream, key / value append to separate paged pools, differential
// attention).  `f32` selects the activation type of the call: float (exact mode) or bf16 (serving); norm weights are always float.
#pragma once
#include <cuda_runtime.h>

namespace b200 {
cudaError_t layernorm_cast_launch(const float* x, long long ld_x, const float* w, const float* b, void* out, bool f32, int n, float eps, int T,
                                  cudaStream_t s);
cudaError_t post_layernorm_add_norm_launch(float* x, const float* y, long long ld_y, const float* pw, const float* pb, float mult, const float* nw,
                                           const float* nb, void* xa, bool f32, int n, float eps, int T, cudaStream_t s);
cudaError_t paged_kv_append_launch(const void* rows, long long ld, int k0, int v0, void* kpool, void* vpool, const int* slot_map, int G, int dk,
                                   int dv, int page, bool f32, int T, cudaStream_t s);
// warps (= query heads) per CTA of the attention kernel for H query heads over G key / value heads
int diff_attention_warps(int H, int G);
// part: fp32 [T, H, nsplit, 2, V + 2] when nsplit > 1 (keys split in chunks of `chunk`, a multiple of 32), else unused
cudaError_t diff_attention_launch(const void* q, long long ld_q, const void* kpool, const void* vpool, const int* block_tables, int max_blocks,
                                  const int* positions, const int* cu, int B, int H, int G, int D, int V, int page, float scale, float softcap,
                                  float temp_coef, float temp_every, float lam, float eps, float out_mult, void* out, bool f32, int T, int nsplit,
                                  int chunk, float* part, cudaStream_t s);
cudaError_t diff_head_norm_launch(const float* a, int T, int H, int G, int V, float lam, float eps, float out_mult, void* out, bool f32,
                                  cudaStream_t s);
}  // namespace b200
