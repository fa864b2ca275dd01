// Kernels of hybrid decoder stacks: recurrent mixers (selective state-space scan, decayed linear attention), the short causal
// convolution in front of them, gated / grouped RMS norms, output-side ("post") norm fused with the fp32 residual add, latent
// multi-query attention with a softmax sink over a paged latent pool, and the small gathers around them.
//
// Conventions: a step is a ragged batch (rows cu_seqlens[b] .. cu_seqlens[b+1] belong to sequence b, whose first row sits at
// position context_lens[b] - q_len); recurrent state lives in per-sequence slots and a sequence whose step starts at position 0
// starts from a zero state whatever its slot holds, so slots are re-used without a clear.  Activations are AT = bf16 (serving) or
// float (exact mode); the residual stream, norms, softmax and every recurrence are fp32 in both.
#include "hybrid.h"
#include "hybrid_common.cuh"

namespace b200 {
namespace {

// ---------------------------------------------------------------------------------------------------------- gathers
template <typename TT, typename OT>
__global__ void gather_rows_kernel(const TT* __restrict__ table, long long ld, const long long* __restrict__ ids, int col0, int n,
                                   OT* __restrict__ out) {
  const long long row = ids[blockIdx.x];
  const TT* src = table + row * ld + col0;
  OT* dst = out + (long long)blockIdx.x * n;
  for (int c = threadIdx.x; c < n; c += blockDim.x) stf<OT>(dst + c, ldf<TT>(src + c));
}

template <typename AT>
__global__ void side_gate_kernel(const AT* __restrict__ gx, long long ld_g, const AT* __restrict__ table, long long ld_t,
                                 const long long* __restrict__ ids, int col0, int n, AT* __restrict__ out) {
  const int t = blockIdx.x;
  const AT* e = table + ids[t] * ld_t + col0;
  for (int c = threadIdx.x; c < n; c += blockDim.x)
    stf<AT>(out + (long long)t * n + c, rnd<AT>(gelu_tanh_f(ldf<AT>(gx + t * ld_g + c))) * ldf<AT>(e + c));
}

template <typename AT>
__global__ void gelu_erf_kernel(AT* __restrict__ x, long long ld, int n) {
  AT* row = x + (long long)blockIdx.x * ld;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) stf<AT>(row + c, gelu_erf_f(ldf<AT>(row + c)));
}

// ---------------------------------------------------------------------------------------------------------- norms
// x += y * rsqrt(mean(y^2) + eps) * w  (x, y fp32);  xa = (AT) x  when xa != nullptr
template <typename AT>
__global__ void post_norm_add_kernel(float* __restrict__ x, const float* __restrict__ y, long long ld_y, const float* __restrict__ w,
                                     AT* __restrict__ xa, int n, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const float* yr = y + t * ld_y;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) { const float v = yr[c]; ss += v * v; }
  const float r = rsqrtf(block_sum(ss, red) / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float v = x[t * n + c] + yr[c] * r * w[c];
    x[t * n + c] = v;
    if (xa != nullptr) stf<AT>(xa + t * n + c, v);
  }
}

template <typename AT>
__global__ void rmsnorm_cast_kernel(const float* __restrict__ x, long long ld_x, const float* __restrict__ w, AT* __restrict__ out, int n,
                                    float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const float* xr = x + t * ld_x;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) { const float v = xr[c]; ss += v * v; }
  const float r = rsqrtf(block_sum(ss, red) / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x) stf<AT>(out + t * n + c, xr[c] * r * w[c]);
}

// mode 0: norm_groups(y * silu(g)) * w      mode 1: norm(y) * w * sigmoid(g)        grid (T, groups)
template <typename AT>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ y, const AT* __restrict__ g, long long ld_g, const float* __restrict__ w,
                                     AT* __restrict__ out, int C, int groups, int mode, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const int gs = C / groups, c0 = blockIdx.y * gs;
  const float* yr = y + t * C + c0;
  const AT* gr = g + t * ld_g + c0;
  float ss = 0.f;
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float v = yr[c];
    if (mode == 0) v *= silu_f(ldf<AT>(gr + c));
    ss += v * v;
  }
  const float r = rsqrtf(block_sum(ss, red) / (float)gs + eps);
  for (int c = threadIdx.x; c < gs; c += blockDim.x) {
    float v = yr[c];
    const float gv = ldf<AT>(gr + c);
    if (mode == 0) v *= silu_f(gv);
    v = v * r * w[c0 + c];
    if (mode == 1) v *= sigmoid_f(gv);
    stf<AT>(out + t * C + c0 + c, v);
  }
}

// ---------------------------------------------------------------------------------------------------------- short convolution
// out[t, c] = silu(b[c] + sum_k w[c, k] * in(t - (K-1) + k, c)); inputs before this step come from the sequence's conv state
// ([slots, K-1, C], the last K-1 inputs), inputs before position 0 are zero.          grid (T, ceil(C / blockDim))
template <typename AT>
__global__ void causal_conv_silu_kernel(const AT* __restrict__ u, long long ld_u, const float* __restrict__ w, const float* __restrict__ bias,
                                        const AT* __restrict__ cstate, const int* __restrict__ cu, const int* __restrict__ ctx,
                                        const int* __restrict__ slots, int B, int C, int K, AT* __restrict__ out) {
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = seq_of(cu, B, t);
  const int j = t - cu[b], c0 = ctx[b] - (cu[b + 1] - cu[b]);
  const AT* st = cstate + (long long)slots[b] * (K - 1) * C;
  float acc = bias[c];
  for (int k = 0; k < K; ++k) {
    const int jj = j - (K - 1) + k;          // row of this step (>= 0) or history (< 0)
    float v = 0.f;
    if (jj >= 0) v = ldf<AT>(u + (long long)(t - j + jj) * ld_u + c);
    else if (c0 > 0) v = ldf<AT>(st + (long long)(K - 1 + jj) * C + c);
    acc += w[c * K + k] * v;
  }
  stf<AT>(out + (long long)t * C + c, silu_f(rnd<AT>(acc)));
}

// new state = last K-1 inputs of the sequence; each thread owns one (sequence, channel) column: reads, then writes
template <typename AT>
__global__ void conv_state_update_kernel(const AT* __restrict__ u, long long ld_u, AT* __restrict__ cstate, const int* __restrict__ cu,
                                         const int* __restrict__ ctx, const int* __restrict__ slots, int C, int K) {
  const int b = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int s = cu[b], q = cu[b + 1] - s, c0 = ctx[b] - q;
  if (q == 0) return;
  AT* st = cstate + (long long)slots[b] * (K - 1) * C;
  float keep[16];
  for (int i = 0; i < K - 1; ++i) {
    const int jj = q - (K - 1) + i;
    float v = 0.f;
    if (jj >= 0) v = ldf<AT>(u + (long long)(s + jj) * ld_u + c);
    else if (c0 > 0 && c0 + jj >= 0) v = ldf<AT>(st + (long long)(K - 1 + jj) * C + c);
    keep[i] = v;
  }
  for (int i = 0; i < K - 1; ++i) stf<AT>(st + (long long)i * C + c, keep[i]);
}

// ---------------------------------------------------------------------------------------------------------- recurrent scans
// One CTA per (sequence, head); state S[N][P] in shared memory (fp32), thread (r, p) owns rows n = r, r + R, ... of column p.
//   MODE 0 (selective state space):  a_t = exp(-exp(A_log) dt_t), S <- a_t S + (dt_t B_t[n]) x_t[p], y_t[p] = sum_n S C_t[n] + D x_t[p]
//   MODE 1 (decayed linear attention): S <- decay S + silu(k_t)[n] silu(v_t)[p], o_t[p] = sum_n S silu(q_t)[n]
struct ScanArgs {
  const void* in; long long ld_in;       // MODE 0: conv output [x | B | C];  MODE 1: projection [q | k | v | ...]
  const void* dt; long long ld_dt;       // MODE 0: raw step sizes [T, H]
  const float* dt_bias; const float* A_log; const float* D; const float* decay;
  float* state;                          // [slots, H, N, P]
  const int* cu; const int* ctx; const int* slots;
  float* out;                            // fp32 [T, H * P]
  int H, N, P, G;
};

constexpr int kScanTokensMax = 16;   // tokens whose operands are staged in shared memory at a time (fewer for decode steps)

template <typename AT, int MODE>
__global__ void recurrent_scan_kernel(ScanArgs a, int PB, int kScanTokens) {
  extern __shared__ float smem[];
  const int b = blockIdx.x, h = blockIdx.y, N = a.N, P = a.P, H = a.H, p0 = blockIdx.z * PB;
  const int R = blockDim.x / PB, p = threadIdx.x % PB, r = threadIdx.x / PB;
  float* S = smem;                          // [N][PB]   this CTA's columns p0 .. p0 + PB of the head's state
  float* red = S + N * PB;                  // [2][R][PB]
  float* kq = red + 2 * R * PB;             // [tokens][2N]  k (already scaled) | q
  float* xs = kq + kScanTokens * 2 * N;     // [tokens][PB]
  float* dc = xs + kScanTokens * PB;        // [tokens]      decay
  float* dts = dc + kScanTokens;            // [tokens]      step size
  const int s = a.cu[b], q = a.cu[b + 1] - s;
  if (q == 0) return;
  const bool fresh = a.ctx[b] - q == 0;
  float* gs = a.state + ((long long)a.slots[b] * H + h) * N * P;
  const int rows_pass = blockDim.x / PB;     // rows of the state block copied per pass (thread (r, p) copies column p)
  if (r < rows_pass)
    for (int n = r; n < N; n += rows_pass) S[n * PB + p] = fresh ? 0.f : gs[n * P + p0 + p];
  const AT* in = reinterpret_cast<const AT*>(a.in);
  const int g = MODE == 0 ? h / (H / a.G) : 0;
  const float Aneg = MODE == 0 ? -expf(a.A_log[h]) : 0.f, Dh = MODE == 0 ? a.D[h] : 0.f, dtb = MODE == 0 ? a.dt_bias[h] : 0.f;
  const float dec = MODE == 1 ? a.decay[h] : 0.f;
  for (int j0 = 0; j0 < q; j0 += kScanTokens) {
    const int nt = min(kScanTokens, q - j0);
    __syncthreads();                        // the last block's operands are no longer read (and S is loaded)
    if (MODE == 0) {                        // per-token step size and decay, once
      for (int jj = threadIdx.x; jj < nt; jj += blockDim.x) {
        const float dt = softplus_f(ldf<AT>(reinterpret_cast<const AT*>(a.dt) + (long long)(s + j0 + jj) * a.ld_dt + h) + dtb);
        dts[jj] = dt;
        dc[jj] = expf(Aneg * dt);
      }
      __syncthreads();
    }
    for (int e = threadIdx.x; e < 2 * N + PB; e += blockDim.x) {
      // each thread owns operand columns e: its source column in the input row is fixed, the loads of the staged tokens are independent
      int col;
      if (MODE == 0) col = e < N ? H * P + g * N + e : (e < 2 * N ? H * P + a.G * N + g * N + (e - N) : h * P + p0 + (e - 2 * N));
      else col = e < N ? H * N + h * N + e : (e < 2 * N ? h * N + (e - N) : 2 * H * N + h * P + p0 + (e - 2 * N));
      const AT* src = in + (long long)(s + j0) * a.ld_in + col;
#pragma unroll 4
      for (int jj = 0; jj < nt; ++jj) {
        float v = ldf<AT>(src + (long long)jj * a.ld_in);
        if (MODE == 1) v = silu_f(v);
        else if (e < N) v *= dts[jj];
        if (e < 2 * N) kq[jj * 2 * N + e] = v;
        else xs[jj * PB + e - 2 * N] = v;
      }
    }
    __syncthreads();
    for (int jj = 0; jj < nt; ++jj) {
      const int j = j0 + jj;
      const float decay = MODE == 0 ? dc[jj] : dec, xv = xs[jj * PB + p];
      const float* kr = kq + jj * 2 * N;
      if (r < R) {
        float acc = 0.f;
        for (int n = r; n < N; n += R) {
          const float sv = decay * S[n * PB + p] + kr[n] * xv;
          S[n * PB + p] = sv;
          acc += sv * kr[N + n];
        }
        red[((j & 1) * R + r) * PB + p] = acc;
      }
      __syncthreads();
      if (r == 0) {
        float y = 0.f;
        for (int i = 0; i < R; ++i) y += red[((j & 1) * R + i) * PB + p];
        a.out[(long long)(s + j) * H * P + h * P + p0 + p] = y + Dh * xv;
      }
    }
  }
  __syncthreads();
  if (r < rows_pass)
    for (int n = r; n < N; n += rows_pass) gs[n * P + p0 + p] = S[n * PB + p];
}

// ---------------------------------------------------------------------------------------------------------- latent attention
// row [c_q raw: Qr | c raw: L | k_rot raw: R]  ->  cq = rms(c_q) * qn_w ;  pool[slot] = [rms(c) * kvn_w | rotate(k_rot, pos)]
template <typename AT>
__global__ void latent_prologue_kernel(const AT* __restrict__ x, long long ld_x, int Qr, int L, int R, const float* __restrict__ qn_w,
                                       const float* __restrict__ kvn_w, float eps, AT* __restrict__ cq, AT* __restrict__ pool,
                                       const int* __restrict__ slot_map, const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                       int interleaved) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const AT* row = x + t * ld_x;
  float ss = 0.f, r;
  if (Qr > 0) {     // Qr == 0: a design without a query latent
    for (int c = threadIdx.x; c < Qr; c += blockDim.x) { const float v = ldf<AT>(row + c); ss += v * v; }
    r = rsqrtf(block_sum(ss, red) / (float)Qr + eps);
    for (int c = threadIdx.x; c < Qr; c += blockDim.x) stf<AT>(cq + t * Qr + c, ldf<AT>(row + c) * r * qn_w[c]);
  }
  ss = 0.f;
  for (int c = threadIdx.x; c < L; c += blockDim.x) { const float v = ldf<AT>(row + Qr + c); ss += v * v; }
  r = rsqrtf(block_sum(ss, red) / (float)L + eps);
  AT* dst = pool + (long long)slot_map[t] * (L + R);
  for (int c = threadIdx.x; c < L; c += blockDim.x) stf<AT>(dst + c, ldf<AT>(row + Qr + c) * r * kvn_w[c]);
  const float pos = (float)positions[t];
  const int half = R / 2;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    sincosf(pos * inv_freq[i], &sn, &cs);
    const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : half + i;     // pair (2i, 2i+1) or (i, i + R/2)
    const float u = ldf<AT>(row + Qr + L + iu), v = ldf<AT>(row + Qr + L + iv);
    stf<AT>(dst + L + iu, u * cs - v * sn);
    stf<AT>(dst + L + iv, v * cs + u * sn);
  }
}

// Causal multi-query attention over the paged latent rows, with a sink: softmax denominator = exp(sink_h) + sum_j exp(s_j).
// grid (T, ceil(H / warps)); one warp per head; key tiles of 32 rows staged in shared memory as fp32 and shared by the heads.
constexpr int kLatTile = 32;
constexpr int kLatMaxPerLane = 32;   // output registers per lane: 16 for a latent width <= 512, 32 up to 1024

// VEC (kv_rank a multiple of 128, row width a multiple of 4): 16-byte shared-memory loads in both phases — lane l owns output dims
// 4l + 128i .. +3 — and key rows padded to a multiple of 4 floats; otherwise scalar loads, lane l owns dims l + 32i, rows padded by 1.
template <typename AT, bool VEC, int NPL>
__global__ void latent_attention_kernel(const AT* __restrict__ q, const AT* __restrict__ pool, const float* __restrict__ sink,
                                        const int* __restrict__ block_tables, int max_blocks, const int* __restrict__ positions,
                                        const int* __restrict__ cu, int B, int H, int L, int R, int page, float scale,
                                        const float* __restrict__ inv_freq, AT* __restrict__ out, int nsplit, int chunk,
                                        float* __restrict__ part, int window, int interleaved) {
  extern __shared__ float smem[];
  const int Dq = L + R, ldk = VEC ? Dq + 4 : Dq + 1, nw = blockDim.x >> 5;
  float* qs = smem;                       // [nw][Dq]
  float* ks = smem + nw * Dq;             // [tile][Dq + 1]
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y * nw + warp;
  const int pos = positions[t];
  const int b = seq_of(cu, B, t);
  const int* bt = block_tables + (long long)b * max_blocks;
  // queries of this block's heads -> smem (rot part rotated by the token's position)
  const int half = R / 2;
  for (int i = threadIdx.x; i < nw * Dq; i += blockDim.x) {
    const int hh = blockIdx.y * nw + i / Dq, d = i % Dq;
    float v = 0.f;
    if (hh < H) {
      const AT* qr = q + ((long long)t * H + hh) * Dq;
      if (d < L) v = ldf<AT>(qr + d);
      else {
        const int e = d - L, f = interleaved ? e >> 1 : (e < half ? e : e - half);
        const bool first = interleaved ? (e & 1) == 0 : e < half;
        float sn, cs;
        sincosf((float)pos * inv_freq[f], &sn, &cs);
        const float u = ldf<AT>(qr + L + (interleaved ? 2 * f : f)), w = ldf<AT>(qr + L + (interleaved ? 2 * f + 1 : half + f));
        v = rnd<AT>(first ? u * cs - w * sn : w * cs + u * sn);
      }
    }
    qs[i] = v;
  }
  // the sink: one extra term exp(sink - m) of the denominator, no key, no value (added by the combine kernel when keys are split)
  // (sink == nullptr: the ordinary softmax.)  window > 0: only keys pos - window < j <= pos are visible; key splits count from the
  // first visible key of this token
  const bool has_sink = sink != nullptr && nsplit == 1;
  float m = has_sink ? (h < H ? sink[h] : 0.f) : -INFINITY, l = has_sink ? 1.f : 0.f;
  const int jlo = window > 0 ? max(0, pos - window + 1) : 0;
  float o[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) o[i] = 0.f;
  const int nper = (L + 31) / 32;
  const float* qh = qs + warp * Dq;
  const int jend = (int)min((long long)pos + 1, (long long)jlo + (long long)(blockIdx.z + 1) * chunk);
  for (int j0 = jlo + blockIdx.z * chunk; j0 < jend; j0 += kLatTile) {
    __syncthreads();
    const int nk = min(kLatTile, jend - j0);
    // each warp fetches whole rows: 16-byte chunks per lane (several independent loads in flight), one block-table lookup per row
    for (int jj = warp; jj < nk; jj += nw) {
      const int j = j0 + jj;
      const AT* src = pool + ((long long)bt[j / page] * page + j % page) * Dq;
      float* dst = ks + jj * ldk;
      constexpr int E = 16 / (int)sizeof(AT);
      if (Dq % E == 0) {
        for (int c = lane; c < Dq / E; c += 32) {
          const uint4 v = *reinterpret_cast<const uint4*>(src + c * E);
          if (VEC) {
            float f[E];
            unpack16<AT>(v, f);
#pragma unroll
            for (int e = 0; e < E; e += 4) *reinterpret_cast<float4*>(dst + c * E + e) = make_float4(f[e], f[e + 1], f[e + 2], f[e + 3]);
          } else {
            unpack16<AT>(v, dst + c * E);
          }
        }
      } else {
        for (int d = lane; d < Dq; d += 32) dst[d] = ldf<AT>(src + d);
      }
    }
    __syncthreads();
    if (h >= H) continue;
    float sc = -INFINITY;
    if (lane < nk) {
      const float* kr = ks + lane * ldk;
      float acc = 0.f;
      if (VEC) {
        const float4* q4 = reinterpret_cast<const float4*>(qh);
        const float4* k4 = reinterpret_cast<const float4*>(kr);
        for (int d = 0; d < Dq / 4; ++d) {
          const float4 a = q4[d], b = k4[d];
          acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
        }
      } else {
        for (int d = 0; d < Dq; ++d) acc += qh[d] * kr[d];
      }
      sc = acc * scale;
    }
    const float mn = fmaxf(m, warp_max(sc));
    const float corr = m == -INFINITY ? 0.f : expf(m - mn), pj = lane < nk ? expf(sc - mn) : 0.f;
    l = l * corr + warp_sum(pj);
    m = mn;
#pragma unroll
    for (int i = 0; i < NPL; ++i) o[i] *= corr;
    for (int jj = 0; jj < nk; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const float* kr = ks + jj * ldk;
      if (VEC) {
#pragma unroll
        for (int i = 0; i < NPL / 4; ++i)
          if (i < L / 128) {
            const float4 c = *reinterpret_cast<const float4*>(kr + 4 * lane + 128 * i);
            o[4 * i] += pv * c.x; o[4 * i + 1] += pv * c.y; o[4 * i + 2] += pv * c.z; o[4 * i + 3] += pv * c.w;
          }
      } else {
#pragma unroll
        for (int i = 0; i < NPL; ++i)
          if (i < nper) { const int d = lane + 32 * i; if (d < L) o[i] += pv * kr[d]; }
      }
    }
  }
  // register i of a lane holds output dim: VEC 4 lane + 128 (i / 4) + i % 4, else lane + 32 i
  if (h < H && nsplit == 1) {
    const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = VEC ? 4 * lane + 128 * (i / 4) + (i % 4) : lane + 32 * i;
      if (d < L) stf<AT>(out + ((long long)t * H + h) * L + d, o[i] * inv);
    }
  } else if (h < H) {
    float* pp = part + (((long long)t * H + h) * nsplit + blockIdx.z) * (L + 2);
    if (lane == 0) { pp[0] = m; pp[1] = l; }
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = VEC ? 4 * lane + 128 * (i / 4) + (i % 4) : lane + 32 * i;
      if (d < L) pp[2 + d] = o[i];
    }
  }
}

// merge the key splits of one (token, head): out = sum_z o_z e^(m_z - M) / (e^(sink - M) + sum_z l_z e^(m_z - M))
template <typename AT>
__global__ void latent_combine_kernel(const float* __restrict__ part, const float* __restrict__ sink, int H, int L, int nsplit,
                                      AT* __restrict__ out) {
  const long long th = blockIdx.x;
  const float* pp = part + th * nsplit * (L + 2);
  const float sk = sink != nullptr ? sink[th % H] : -INFINITY;
  float M = sk;
  for (int z = 0; z < nsplit; ++z) M = fmaxf(M, pp[z * (L + 2)]);
  float den = sink != nullptr ? expf(sk - M) : 0.f;
  for (int z = 0; z < nsplit; ++z) { const float mz = pp[z * (L + 2)]; if (mz != -INFINITY) den += pp[z * (L + 2) + 1] * expf(mz - M); }
  for (int d = threadIdx.x; d < L; d += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < nsplit; ++z) { const float mz = pp[z * (L + 2)]; if (mz != -INFINITY) acc += pp[z * (L + 2) + 2 + d] * expf(mz - M); }
    stf<AT>(out + th * L + d, acc / den);
  }
}


// ---- prefill of one sequence as two GEMMs: scores = Q K^T and out = P C (library / tcgen05 GEMMs) around these two kernels
// rotate-half rotary, in place, on dims [L, L + R) of every head of q [T, H, L + R]
template <typename AT>
__global__ void rotate_half_kernel(AT* __restrict__ q, const int* __restrict__ positions, const float* __restrict__ inv_freq, int H, int L,
                                   int R, int interleaved) {
  const int t = blockIdx.x, half = R / 2;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
    const int h = i / half, f = i % half;
    AT* p = q + ((long long)t * H + h) * (L + R) + L;
    float sn, cs;
    sincosf(pos * inv_freq[f], &sn, &cs);
    const int iu = interleaved ? 2 * f : f, iv = interleaved ? 2 * f + 1 : half + f;
    const float u = ldf<AT>(p + iu), v = ldf<AT>(p + iv);
    stf<AT>(p + iu, u * cs - v * sn);
    stf<AT>(p + iv, v * cs + u * sn);
  }
}

// row r = (token t, head h) of raw scores [rows, n]; column j is the key at position k0 + j; the query sits at position ctx0 + t and sees
// keys at positions <= its own (and > its own - window when window > 0); p_j = e^(s_j scale - m) / (e^(sink_h - m) + sum), the sink
// term only when sink != nullptr.  temp_coef != 0: the query's scores are multiplied by 1 + temp_coef ln(floor((qp + 1) / temp_every) + 1);
// softcap > 0: s <- softcap tanh(s / softcap) after the scaling
struct ScoreMap {
  float scale, softcap;
  __device__ __forceinline__ float operator()(float v) const { v *= scale; return softcap > 0.f ? softcap * tanhf(v / softcap) : v; }
};
template <typename AT>
__global__ void sink_softmax_kernel(const float* __restrict__ s, const float* __restrict__ sink, int H, int n, int ctx0, float scale0,
                                    AT* __restrict__ out, int window, int k0, float softcap, float temp_coef, float temp_every) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  const int t = (int)(r / H), h = (int)(r % H), qp = ctx0 + t;
  const ScoreMap f{temp_coef != 0.f ? scale0 * (1.f + temp_coef * logf(floorf((float)(qp + 1) / temp_every) + 1.f)) : scale0, softcap};
  const int nv = max(0, min(n, qp - k0 + 1)), j_lo = window > 0 ? max(0, qp - window + 1 - k0) : 0;
  const float* row = s + r * n;
  const float sk = sink != nullptr ? sink[h] : -INFINITY;
  float m = sk;
  for (int j = j_lo + threadIdx.x; j < nv; j += blockDim.x) m = fmaxf(m, f(row[j]));
  m = warp_max(m);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (l == 0) red[w] = m;
  __syncthreads();
  m = warp_max(l < nw ? red[l] : -INFINITY);
  float sum = 0.f;
  for (int j = j_lo + threadIdx.x; j < nv; j += blockDim.x) sum += expf(f(row[j]) - m);
  const float inv = 1.f / (block_sum(sum, red) + (sink != nullptr ? expf(sk - m) : 0.f));
  for (int j = threadIdx.x; j < n; j += blockDim.x) stf<AT>(out + r * n + j, (j >= j_lo && j < nv) ? expf(f(row[j]) - m) * inv : 0.f);
}

// ---------------------------------------------------------------------------------------------------------- pre-norm residual step
// x += (y + extra * sigmoid(gate[t])) * ls   (x, y, extra fp32; ls, extra nullable);   xa = (AT)(x * rsqrt(mean(x^2) + eps) * w)
template <typename AT>
__global__ void scaled_add_norm_kernel(float* __restrict__ x, const float* __restrict__ y, long long ld_y, const float* __restrict__ ls,
                                       const float* __restrict__ extra, long long ld_e, const float* __restrict__ gate, long long ld_gate,
                                       const float* __restrict__ w, AT* __restrict__ xa, int n, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const float* yr = y + t * ld_y;
  const float* er = extra != nullptr ? extra + t * ld_e : nullptr;
  const float sg = extra != nullptr ? sigmoid_f(gate[t * ld_gate]) : 0.f;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    float v = yr[c];
    if (er != nullptr) v += er[c] * sg;
    if (ls != nullptr) v *= ls[c];
    v += x[t * n + c];
    x[t * n + c] = v;
    ss += v * v;
  }
  const float r = rsqrtf(block_sum(ss, red) / (float)n + eps);
  for (int c = threadIdx.x; c < n; c += blockDim.x) stf<AT>(xa + t * n + c, x[t * n + c] * r * w[c]);   // own writes: same thread, same c
}

// ---------------------------------------------------------------------------------------------------------- mLSTM scan
// Matrix memory with exponential gating, stabilised by a running maximum m (all fp32):
//   i = cap tanh((gi + bi) / cap), f = logsigmoid(cap tanh((gf + bf) / cap)), m' = max(f + m, i), a = e^(f + m - m'), b = e^(i - m')
//   S <- a S + b k v^T,  n <- a n + b k,  o = S^T q / (max(|n . q|, e^(-m')) + 1e-6);   S, n, m start at zero.
// One CTA per (sequence, head, block of PB value columns); S[N][PB] and n[N] in shared memory.  The normaliser n and the maximum m do
// not depend on the value column, so every column block keeps its OWN copy of them in the state (no CTA reads what another writes).
struct MlstmArgs {
  const void* in; long long ld_in;        // [q: H*N | k: H*N | v: H*P | ...] activations
  const float* gates; long long ld_g;     // raw [gi: H | gf: H] fp32
  const float* gate_bias;                 // [2H]
  float* S; float* n; float* m;           // [slots, H, N, P], [slots, H, P/PB, N], [slots, H, P/PB]
  const int* cu; const int* ctx; const int* slots;
  float* out;                             // fp32 [T, H * P]
  int H, N, P;
  float cap, q_scale;
};

__device__ __forceinline__ float logsigmoid_f(float v) { return fminf(v, 0.f) - log1pf(expf(-fabsf(v))); }

template <typename AT>
__global__ void mlstm_scan_kernel(MlstmArgs a, int PB, int R, int kTok) {
  extern __shared__ float smem[];
  const int b = blockIdx.x, h = blockIdx.y, N = a.N, P = a.P, H = a.H, NB = P / PB, p0 = blockIdx.z * PB;
  const int p = threadIdx.x % PB, r = threadIdx.x / PB, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  float* S = smem;                          // [N][PB]
  float* nv = S + N * PB;                   // [N]
  float* red = nv + N;                      // [2][R][PB]
  float* redn = red + 2 * R * PB;           // [2][32]
  float* kq = redn + 64;                    // [tokens][2N]   b k | q_scale q
  float* xs = kq + kTok * 2 * N;            // [tokens][PB]
  float* da = xs + kTok * PB;               // [tokens] a        (log first, then the exponential)
  float* db = da + kTok;                    // [tokens] b
  float* dm = db + kTok;                    // [tokens] e^(-m')
  float* gi = dm + kTok;                    // [tokens]
  float* gf = gi + kTok;                    // [tokens]
  float* mrun = gf + kTok;                  // [1]
  const int s = a.cu[b], q = a.cu[b + 1] - s;
  if (q == 0) return;
  const bool fresh = a.ctx[b] - q == 0;
  const long long sh = (long long)a.slots[b] * H + h;
  float* gS = a.S + sh * N * P;
  float* gn = a.n + (sh * NB + blockIdx.z) * N;
  float* gm = a.m + sh * NB + blockIdx.z;
  for (int e = threadIdx.x; e < N * PB; e += blockDim.x) { const int n = e / PB, c = e % PB; S[e] = fresh ? 0.f : gS[n * P + p0 + c]; }
  for (int e = threadIdx.x; e < N; e += blockDim.x) nv[e] = fresh ? 0.f : gn[e];
  if (threadIdx.x == 0) mrun[0] = fresh ? 0.f : gm[0];
  const AT* in = reinterpret_cast<const AT*>(a.in);
  const float bi = a.gate_bias[h], bf = a.gate_bias[H + h], cap = a.cap;
  for (int j0 = 0; j0 < q; j0 += kTok) {
    const int nt = min(kTok, q - j0);
    __syncthreads();                        // the last block's operands are no longer read (and the state is loaded)
    for (int jj = threadIdx.x; jj < nt; jj += blockDim.x) {
      const float* g = a.gates + (long long)(s + j0 + jj) * a.ld_g;
      gi[jj] = cap * tanhf((g[h] + bi) / cap);
      gf[jj] = logsigmoid_f(cap * tanhf((g[H + h] + bf) / cap));
    }
    __syncthreads();
    if (threadIdx.x == 0) {                 // the running maximum is a scalar chain: additions and maxima only
      float m = mrun[0];
      for (int jj = 0; jj < nt; ++jj) {
        const float mn = fmaxf(gf[jj] + m, gi[jj]);
        da[jj] = gf[jj] + m - mn; db[jj] = gi[jj] - mn; dm[jj] = -mn;
        m = mn;
      }
      mrun[0] = m;
    }
    __syncthreads();
    for (int jj = threadIdx.x; jj < nt; jj += blockDim.x) { da[jj] = expf(da[jj]); db[jj] = expf(db[jj]); dm[jj] = expf(dm[jj]); }
    __syncthreads();
    for (int e = threadIdx.x; e < 2 * N + PB; e += blockDim.x) {
      const int col = e < N ? H * N + h * N + e : (e < 2 * N ? h * N + (e - N) : 2 * H * N + h * P + p0 + (e - 2 * N));
      const AT* src = in + (long long)(s + j0) * a.ld_in + col;
#pragma unroll 4
      for (int jj = 0; jj < nt; ++jj) {
        float v = ldf<AT>(src + (long long)jj * a.ld_in);
        if (e < N) v *= db[jj];
        else if (e < 2 * N) v *= a.q_scale;
        if (e < 2 * N) kq[jj * 2 * N + e] = v;
        else xs[jj * PB + e - 2 * N] = v;
      }
    }
    __syncthreads();
    for (int jj = 0; jj < nt; ++jj) {
      const int j = j0 + jj;
      const float decay = da[jj], xv = xs[jj * PB + p];
      const float* kr = kq + jj * 2 * N;
      if (r < R) {
        float acc = 0.f;
        for (int n = r; n < N; n += R) {
          const float sv = decay * S[n * PB + p] + kr[n] * xv;
          S[n * PB + p] = sv;
          acc += sv * kr[N + n];
        }
        red[((j & 1) * R + r) * PB + p] = acc;
      }
      float pn = 0.f;                       // normaliser: element e of n belongs to thread e % blockDim
      for (int e = threadIdx.x; e < N; e += blockDim.x) {
        const float nn = decay * nv[e] + kr[e];
        nv[e] = nn;
        pn += nn * kr[N + e];
      }
      pn = warp_sum(pn);
      if (lane == 0) redn[(j & 1) * 32 + warp] = pn;
      __syncthreads();
      if (r == 0) {
        float y = 0.f, nq = 0.f;
        for (int i = 0; i < R; ++i) y += red[((j & 1) * R + i) * PB + p];
        for (int i = 0; i < nw; ++i) nq += redn[(j & 1) * 32 + i];
        a.out[(long long)(s + j) * H * P + h * P + p0 + p] = y / (fmaxf(fabsf(nq), dm[jj]) + 1e-6f);
      }
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < N * PB; e += blockDim.x) { const int n = e / PB, c = e % PB; gS[n * P + p0 + c] = S[e]; }
  for (int e = threadIdx.x; e < N; e += blockDim.x) gn[e] = nv[e];
  if (threadIdx.x == 0) gm[0] = mrun[0];
}

// ---------------------------------------------------------------------------------------------------------- mixture of experts
// Router on fp32 logits, the `top` largest scores (ties: lowest id).  One warp per token.  mode 0: scores sigmoid(z), weights = the chosen
// scores; mode 1: scores z + bias (bias nullable), weights = softmax over the chosen scores alone.
__global__ void sigmoid_topk_kernel(const float* __restrict__ z, long long ld_z, const float* __restrict__ bias, int mode, int E, int top,
                                    int* __restrict__ idx, float* __restrict__ w) {
  extern __shared__ float sc[];             // [E]
  const long long t = blockIdx.x;
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) sc[e] = mode == 0 ? sigmoid_f(z[t * ld_z + e]) : z[t * ld_z + e] + (bias != nullptr ? bias[e] : 0.f);
  __syncwarp();
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) { const float v = sc[e]; if (v > best) { best = v; bi = e; } }   // ascending e: first maximum wins
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { idx[t * top + j] = bi; w[t * top + j] = best; sc[bi] = -INFINITY; }
    __syncwarp();
  }
  if (mode == 1 && lane == 0) {             // the first chosen score is the largest
    const float m = w[t * top];
    float sum = 0.f;
    for (int j = 0; j < top; ++j) sum += expf(w[t * top + j] - m);
    for (int j = 0; j < top; ++j) w[t * top + j] = expf(w[t * top + j] - m) / sum;
  }
}

// gate rows g and up rows u (F wide each, own row strides) -> g' sigmoid(1.702 g') (u' + 1),  g' = min(s g, limit), u' = clamp(s u, +-limit).  Block i handles row
// row_of[i] with scale s = scale[i] (both nullable: row i, scale 1): scaling a projection's output equals scaling its input.
// kind 1: silu(g) u s instead (no clamp; the scale multiplies the product, i.e. the input of the down projection).
template <typename AT>
__global__ void clamped_glu_kernel(const AT* __restrict__ gp, long long ld_g, const AT* __restrict__ up, long long ld_u, int F, float limit,
                                   const int* __restrict__ row_of, const float* __restrict__ scale, AT* __restrict__ out, int kind) {
  const long long r = row_of != nullptr ? row_of[blockIdx.x] : blockIdx.x;
  const float s = scale != nullptr ? scale[blockIdx.x] : 1.f;
  const AT* grow = gp + r * ld_g;
  const AT* urow = up + r * ld_u;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < F; c += gridDim.y * blockDim.x) {
    if (kind == 1) { stf<AT>(out + r * F + c, silu_f(ldf<AT>(grow + c)) * ldf<AT>(urow + c) * s); continue; }
    const float g = fminf(s * ldf<AT>(grow + c), limit), u = fminf(fmaxf(s * ldf<AT>(urow + c), -limit), limit);
    stf<AT>(out + r * F + c, g * sigmoid_f(1.702f * g) * (u + 1.f));
  }
}

// out[i, n] = sum_k x[src(i), k] * W[expert[i], n, k]  (fp32 accumulate): one weight bank row per warp, every row with its own expert.
// src(i) = i / div (div = top-k when x holds one row per token and i counts (token, choice) pairs).  Exact-mode and odd-size path of
// the routed experts; no host involvement, so it can sit in a captured graph.        grid (rows, ceil(N / warps))
template <typename AT, typename OT>
__global__ void expert_rows_linear_kernel(const AT* __restrict__ x, long long ld_x, int div, const AT* __restrict__ W, const int* __restrict__ expert,
                                          int N, int K, OT* __restrict__ out) {
  const long long i = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = blockIdx.y * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const AT* xr = x + (i / div) * ld_x;
  const AT* wr = W + ((long long)expert[i] * N + n) * K;
  float acc = 0.f;
  for (int k = lane; k < K; k += 32) acc += ldf<AT>(xr + k) * ldf<AT>(wr + k);
  acc = warp_sum(acc);
  if (lane == 0) stf<OT>(out + i * N + n, acc);
}

// out[t] = sum_j wts[t * k + j] y[row_of[t * k + j]]   (fp32; wts nullable: 1; row_of nullable: row t * k + j): the routed experts' results
// back in token order
__global__ void gather_sum_kernel(const float* __restrict__ y, const int* __restrict__ row_of, const float* __restrict__ wts, int k, int n,
                                  float* __restrict__ out) {
  const long long t = blockIdx.x;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < k; ++j) {
      const long long r = row_of != nullptr ? row_of[t * k + j] : t * k + j;
      acc += (wts != nullptr ? wts[t * k + j] : 1.f) * y[r * n + c];
    }
    out[t * n + c] = acc;
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------- launchers
cudaError_t gather_rows_launch(const void* table, bool table_f32, long long ld, const long long* ids, int col0, int n, void* out,
                               bool out_f32, int T, cudaStream_t s) {
  const int th = n >= 256 ? 256 : 64;
  if (table_f32 && out_f32) gather_rows_kernel<float, float><<<T, th, 0, s>>>((const float*)table, ld, ids, col0, n, (float*)out);
  else if (table_f32) gather_rows_kernel<float, __nv_bfloat16><<<T, th, 0, s>>>((const float*)table, ld, ids, col0, n, (__nv_bfloat16*)out);
  else if (out_f32) gather_rows_kernel<__nv_bfloat16, float><<<T, th, 0, s>>>((const __nv_bfloat16*)table, ld, ids, col0, n, (float*)out);
  else gather_rows_kernel<__nv_bfloat16, __nv_bfloat16><<<T, th, 0, s>>>((const __nv_bfloat16*)table, ld, ids, col0, n, (__nv_bfloat16*)out);
  return last();
}

cudaError_t side_gate_launch(const void* gx, long long ld_g, const void* table, long long ld_t, const long long* ids, int col0, int n,
                             void* out, bool f32, int T, cudaStream_t s) {
  AT_DISPATCH(f32, (side_gate_kernel<AT><<<T, 64, 0, s>>>((const AT*)gx, ld_g, (const AT*)table, ld_t, ids, col0, n, (AT*)out)));
  return last();
}

cudaError_t gelu_erf_launch(void* x, long long ld, int n, bool f32, int T, cudaStream_t s) {
  dim3 grid(T, (n + 1023) / 1024);
  AT_DISPATCH(f32, (gelu_erf_kernel<AT><<<grid, 256, 0, s>>>((AT*)x, ld, n)));
  return last();
}

cudaError_t post_norm_add_launch(float* x, const float* y, long long ld_y, const float* w, void* xa, bool f32, int n, float eps, int T,
                                 cudaStream_t s) {
  AT_DISPATCH(f32, (post_norm_add_kernel<AT><<<T, 256, 0, s>>>(x, y, ld_y, w, (AT*)xa, n, eps)));
  return last();
}

cudaError_t rmsnorm_cast_launch(const float* x, long long ld_x, const float* w, void* out, bool f32, int n, float eps, int T,
                                cudaStream_t s) {
  AT_DISPATCH(f32, (rmsnorm_cast_kernel<AT><<<T, 256, 0, s>>>(x, ld_x, w, (AT*)out, n, eps)));
  return last();
}

cudaError_t gated_rmsnorm_launch(const float* y, const void* g, long long ld_g, const float* w, void* out, bool f32, int C, int groups,
                                 int mode, float eps, int T, cudaStream_t s) {
  dim3 grid(T, groups);
  AT_DISPATCH(f32, (gated_rmsnorm_kernel<AT><<<grid, 256, 0, s>>>(y, (const AT*)g, ld_g, w, (AT*)out, C, groups, mode, eps)));
  return last();
}

cudaError_t causal_conv_silu_launch(const void* u, long long ld_u, const float* w, const float* bias, void* cstate, const int* cu,
                                    const int* ctx, const int* slots, int B, int C, int K, void* out, bool f32, int T, cudaStream_t s) {
  if (K - 1 > 16) return cudaErrorInvalidValue;
  dim3 grid(T, (C + 255) / 256), gridu(B, (C + 255) / 256);
  AT_DISPATCH(f32, (causal_conv_silu_kernel<AT><<<grid, 256, 0, s>>>((const AT*)u, ld_u, w, bias, (const AT*)cstate, cu, ctx, slots, B, C, K,
                                                                    (AT*)out)));
  if (K > 1)
    AT_DISPATCH(f32, (conv_state_update_kernel<AT><<<gridu, 256, 0, s>>>((const AT*)u, ld_u, (AT*)cstate, cu, ctx, slots, C, K)));
  return last();
}

template <typename AT, int MODE>
static cudaError_t scan_launch_t(const ScanArgs& a, int B, int max_q, cudaStream_t s) {
  const int P = a.P, N = a.N;
  if (P > 1024) return cudaErrorInvalidValue;
  // columns of the state are independent: split a head's value dimension over CTAs (PB columns each) while the grid is small
  int PB = P;
  while (PB > 16 && PB % 2 == 0 && (long long)B * a.H * (P / PB) < 592) PB /= 2;
  int R = 256 / PB;
  if (R < 1) R = 1;
  if (R > N) R = N;
  const int threads = (R * PB + 31) / 32 * 32;   // tail threads (r >= R) only help with staging and the state copy
  const int stage = max_q < 1 ? 1 : (max_q < kScanTokensMax ? max_q : kScanTokensMax);
  const size_t smem = ((size_t)N * PB + 2 * (size_t)R * PB + (size_t)stage * (2 * N + PB + 2)) * sizeof(float);
  auto k = recurrent_scan_kernel<AT, MODE>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
  }
  k<<<dim3(B, a.H, P / PB), threads, smem, s>>>(a, PB, stage);
  return last();
}

cudaError_t ssm_scan_launch(const void* xbc, long long ld_x, const void* dt, long long ld_dt, const float* dt_bias, const float* A_log,
                            const float* D, float* state, const int* cu, const int* ctx, const int* slots, float* out, int B, int H, int N,
                            int P, int G, bool f32, int max_q, cudaStream_t s) {
  ScanArgs a{xbc, ld_x, dt, ld_dt, dt_bias, A_log, D, nullptr, state, cu, ctx, slots, out, H, N, P, G};
  return f32 ? scan_launch_t<float, 0>(a, B, max_q, s) : scan_launch_t<__nv_bfloat16, 0>(a, B, max_q, s);
}

cudaError_t decay_scan_launch(const void* qkv, long long ld, const float* decay, float* state, const int* cu, const int* ctx,
                              const int* slots, float* out, int B, int H, int N, int P, bool f32, int max_q, cudaStream_t s) {
  ScanArgs a{qkv, ld, nullptr, 0, nullptr, nullptr, nullptr, decay, state, cu, ctx, slots, out, H, N, P, 1};
  return f32 ? scan_launch_t<float, 1>(a, B, max_q, s) : scan_launch_t<__nv_bfloat16, 1>(a, B, max_q, s);
}

cudaError_t latent_prologue_launch(const void* x, long long ld_x, int Qr, int L, int R, const float* qn_w, const float* kvn_w, float eps,
                                   void* cq, void* pool, const int* slot_map, const int* positions, const float* inv_freq, bool f32, int T,
                                   int interleaved, cudaStream_t s) {
  AT_DISPATCH(f32, (latent_prologue_kernel<AT><<<T, 256, 0, s>>>((const AT*)x, ld_x, Qr, L, R, qn_w, kvn_w, eps, (AT*)cq, (AT*)pool, slot_map,
                                                                 positions, inv_freq, interleaved)));
  return last();
}

cudaError_t rotate_half_launch(void* q, const int* positions, const float* inv_freq, int H, int L, int R, bool f32, int T, int interleaved,
                               cudaStream_t s) {
  AT_DISPATCH(f32, (rotate_half_kernel<AT><<<T, 128, 0, s>>>((AT*)q, positions, inv_freq, H, L, R, interleaved)));
  return last();
}

cudaError_t sink_softmax_launch(const float* sc, const float* sink, int H, int n, int ctx0, float scale, void* out, bool f32, long long rows,
                                int window, int k0, float softcap, float temp_coef, float temp_every, cudaStream_t s) {
  AT_DISPATCH(f32, (sink_softmax_kernel<AT><<<(unsigned)rows, 256, 0, s>>>(sc, sink, H, n, ctx0, scale, (AT*)out, window, k0, softcap, temp_coef,
                                                                          temp_every)));
  return last();
}

cudaError_t latent_attention_launch(const void* q, const void* pool, const float* sink, const int* block_tables, int max_blocks,
                                    const int* positions, const int* cu, int B, int H, int L, int R, int page, float scale,
                                    const float* inv_freq, void* out, bool f32, int T, int nsplit, int chunk, float* part, int window,
                                    int interleaved, cudaStream_t s) {
  if (L > 32 * kLatMaxPerLane || nsplit < 1 || (nsplit > 1 && part == nullptr)) return cudaErrorInvalidValue;
  const int nw = H < 8 ? H : 8, Dq = L + R;
  const bool vec = L % 128 == 0 && Dq % 4 == 0;
  const size_t smem = ((size_t)nw * Dq + (size_t)kLatTile * (Dq + (vec ? 4 : 1))) * sizeof(float);
  dim3 grid(T, (H + nw - 1) / nw, nsplit);
#define LAT_LAUNCH(AT_, VEC_)                                                                                                          \
  do {                                                                                                                                 \
    auto k = L <= 512 ? latent_attention_kernel<AT_, VEC_, 16> : latent_attention_kernel<AT_, VEC_, 32>;                               \
    if (smem > 48 * 1024) {                                                                                                            \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                                 \
      if (e != cudaSuccess) return e;                                                                                                  \
    }                                                                                                                                  \
    k<<<grid, nw * 32, smem, s>>>((const AT_*)q, (const AT_*)pool, sink, block_tables, max_blocks, positions, cu, B, H, L, R, page, scale, \
                                  inv_freq, (AT_*)out, nsplit, chunk, part, window, interleaved);                                      \
    if (nsplit > 1) latent_combine_kernel<AT_><<<T * H, 128, 0, s>>>(part, sink, H, L, nsplit, (AT_*)out);                             \
  } while (0)
  if (f32) { if (vec) LAT_LAUNCH(float, true); else LAT_LAUNCH(float, false); }
  else { if (vec) LAT_LAUNCH(__nv_bfloat16, true); else LAT_LAUNCH(__nv_bfloat16, false); }
#undef LAT_LAUNCH
  return last();
}

cudaError_t scaled_add_norm_launch(float* x, const float* y, long long ld_y, const float* ls, const float* extra, long long ld_e,
                                   const float* gate, long long ld_gate, const float* w, void* xa, bool f32, int n, float eps, int T,
                                   cudaStream_t s) {
  AT_DISPATCH(f32, (scaled_add_norm_kernel<AT><<<T, 256, 0, s>>>(x, y, ld_y, ls, extra, ld_e, gate, ld_gate, w, (AT*)xa, n, eps)));
  return last();
}

cudaError_t mlstm_scan_launch(const void* in, long long ld_in, const float* gates, long long ld_g, const float* gate_bias, float* S, float* n,
                              float* m, const int* cu, const int* ctx, const int* slots, float* out, int B, int H, int N, int P, int PB,
                              float cap, float q_scale, bool f32, int max_q, cudaStream_t s) {
  if (PB < 1 || P % PB != 0 || PB > 1024) return cudaErrorInvalidValue;
  MlstmArgs a{in, ld_in, gates, ld_g, gate_bias, S, n, m, cu, ctx, slots, out, H, N, P, cap, q_scale};
  int R = 256 / PB;
  if (R < 1) R = 1;
  if (R > N) R = N;
  const int threads = (R * PB + 31) / 32 * 32;   // tail threads (r >= R) help with staging, the normaliser and the state copy
  const int stage = max_q < 1 ? 1 : (max_q < kScanTokensMax ? max_q : kScanTokensMax);
  const size_t smem = ((size_t)N * PB + N + 2 * (size_t)R * PB + 64 + (size_t)stage * (2 * N + PB + 5) + 1) * sizeof(float);
  if (smem > 220 * 1024) return cudaErrorInvalidValue;
  if (f32) {
    auto k = mlstm_scan_kernel<float>;
    if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
    k<<<dim3(B, H, P / PB), threads, smem, s>>>(a, PB, R, stage);
  } else {
    auto k = mlstm_scan_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
    k<<<dim3(B, H, P / PB), threads, smem, s>>>(a, PB, R, stage);
  }
  return last();
}

cudaError_t router_topk_launch(const float* z, long long ld_z, const float* bias, int mode, int E, int top, int* idx, float* w, int T,
                               cudaStream_t s) {
  if (top > E || (size_t)E * sizeof(float) > 48 * 1024) return cudaErrorInvalidValue;
  sigmoid_topk_kernel<<<T, 32, E * sizeof(float), s>>>(z, ld_z, bias, mode, E, top, idx, w);
  return last();
}

cudaError_t clamped_glu_launch(const void* g, long long ld_g, const void* u, long long ld_u, int F, float limit, const int* row_of,
                               const float* scale, void* out, bool f32, int rows, int kind, cudaStream_t s) {
  dim3 grid(rows, (F + 1023) / 1024);
  AT_DISPATCH(f32, (clamped_glu_kernel<AT><<<grid, 256, 0, s>>>((const AT*)g, ld_g, (const AT*)u, ld_u, F, limit, row_of, scale, (AT*)out, kind)));
  return last();
}

cudaError_t expert_rows_linear_launch(const void* x, long long ld_x, int div, const void* W, const int* expert, int N, int K, void* out, bool f32,
                                      bool out_f32, int rows, cudaStream_t s) {
  dim3 grid(rows, (N + 7) / 8);
  if (f32) expert_rows_linear_kernel<float, float><<<grid, 256, 0, s>>>((const float*)x, ld_x, div, (const float*)W, expert, N, K, (float*)out);
  else if (out_f32) expert_rows_linear_kernel<__nv_bfloat16, float><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, ld_x, div, (const __nv_bfloat16*)W, expert, N, K, (float*)out);
  else expert_rows_linear_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, ld_x, div, (const __nv_bfloat16*)W, expert, N, K, (__nv_bfloat16*)out);
  return last();
}

cudaError_t gather_sum_launch(const float* y, const int* row_of, const float* wts, int k, int n, float* out, int T, cudaStream_t s) {
  dim3 grid(T, (n + 1023) / 1024);
  gather_sum_kernel<<<grid, 256, 0, s>>>(y, row_of, wts, k, n, out);
  return last();
}

}  // namespace b200
