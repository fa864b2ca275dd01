// Kernels of stacks that run on several residual streams with dynamic-tanh norms: the stream update fused with the read for the next
// sublayer, the gated delta rule with one decay per head and key channel, grouped-query attention inside fixed blocks of positions
// (or a sliding window) with a sink, its prologue (per-head RMS norm of queries and keys, rotation of adjacent pairs, append to the
// paged pools), minGRU, the group-limited softmax router and the squared ReLU.
//
// Conventions as in hybrid.cu: a step is a ragged batch (rows cu_seqlens[b] .. cu_seqlens[b+1] belong to sequence b, whose recurrent
// state lives in slot slots[b]; a sequence whose step starts at position 0 starts from a zero state); activations are AT = bf16
// (serving) or float (exact mode); streams, norms, scores, softmax, router and everything inside a recurrence are fp32 in both.
#include "streams.h"
#include "hybrid_common.cuh"

namespace b200 {
namespace {

constexpr int kMaxStreams = 8;

// ---------------------------------------------------------------------------------------------------------- streams
// xs[t, s, :] = table[ids[t], :] * scale for every stream s
template <typename TT>
__global__ void stream_embed_kernel(const TT* __restrict__ table, long long ld, const long long* __restrict__ ids, float scale, int S, int n,
                                    float* __restrict__ xs) {
  const long long t = blockIdx.x;
  const TT* row = table + ids[t] * ld;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
    const float v = ldf<TT>(row + c) * scale;
    for (int s = 0; s < S; ++s) xs[(t * S + s) * n + c] = v;
  }
}

struct HyperArgs {
  float* xs;                                // [T, S, n] fp32, updated in place
  const float* y; long long ld_y;           // sublayer output (nullptr: only the read)
  const float* y2; long long ld_y2;         // second branch added to y (nullable)
  const void* gate; long long ld_g;         // gate logits per element, AT (nullable)
  const float* ls;                          // [n] layer scale (nullable)
  const float* mix; const float* out_w;     // [S, S] (from, to), [S]
  const float* in_w;                        // [S] weights of the read that follows
  const float* w; const float* b;           // dynamic tanh of the read: tanh(alpha u) * w + b
  float mult, alpha;
  void* xa;                                 // AT [T, n]
  int S, n;
};

// r = (y + y2) * ls * sigmoid(gate);  xs[t, j] <- sum_s mix[s, j] xs[t, s] + mult * out_w[j] * r;  xa = dyt(sum_j in_w[j] xs[t, j]).
// No row statistics anywhere: every (token, channel) is independent.                      grid (T, ceil(n / blockDim))
template <typename AT>
__global__ void hyper_step_kernel(HyperArgs a) {
  __shared__ float sm[kMaxStreams * kMaxStreams + 2 * kMaxStreams];
  const int S = a.S;
  float* mix = sm; float* ow = sm + kMaxStreams * kMaxStreams; float* iw = ow + kMaxStreams;
  if (threadIdx.x < S * S && a.y != nullptr) mix[threadIdx.x] = a.mix[threadIdx.x];
  if (threadIdx.x < S) { ow[threadIdx.x] = a.y != nullptr ? a.mult * a.out_w[threadIdx.x] : 0.f; iw[threadIdx.x] = a.in_w[threadIdx.x]; }
  __syncthreads();
  const long long t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= a.n) return;
  float* x = a.xs + t * S * a.n + c;
  float old[kMaxStreams], u = 0.f;
#pragma unroll
  for (int s = 0; s < kMaxStreams; ++s) old[s] = s < S ? x[(long long)s * a.n] : 0.f;
  if (a.y != nullptr) {
    float r = a.y[t * a.ld_y + c];
    if (a.y2 != nullptr) r += a.y2[t * a.ld_y2 + c];
    if (a.ls != nullptr) r *= a.ls[c];
    if (a.gate != nullptr) r *= sigmoid_f(ldf<AT>((const AT*)a.gate + t * a.ld_g + c));
#pragma unroll
    for (int j = 0; j < kMaxStreams; ++j) {
      if (j < S) {
        float v = 0.f;
#pragma unroll
        for (int s = 0; s < kMaxStreams; ++s) if (s < S) v += mix[s * S + j] * old[s];
        v += ow[j] * r;
        x[(long long)j * a.n] = v;
        u += iw[j] * v;
      }
    }
  } else {
#pragma unroll
    for (int j = 0; j < kMaxStreams; ++j) if (j < S) u += iw[j] * old[j];
  }
  stf<AT>((AT*)a.xa + t * a.n + c, tanhf(a.alpha * u) * a.w[c] + a.b[c]);
}

template <typename AT>
__global__ void relu2_kernel(AT* __restrict__ x, long long ld, int n) {
  AT* row = x + (long long)blockIdx.x * ld;
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
    const float v = fmaxf(ldf<AT>(row + c), 0.f);
    stf<AT>(row + c, v * v);
  }
}

// ---------------------------------------------------------------------------------------------------------- gated delta rule
struct DeltaArgs {
  const void* in; long long ld_in;          // conv output, AT: [q: G*N | k: G*N | v: H*P]
  const void* beta; long long ld_b;         // raw write strengths, AT [T, >= H]
  const float* dt; long long ld_dt;         // raw step sizes fp32 [T, H*N]
  const float* dt_bias; const float* A_log; // [H*N], [H]
  float* state;                             // [slots, H, N, P]
  const int* cu; const int* ctx; const int* slots;
  float* out;                               // fp32 [T, H*P]
  int H, G, N, P;
  float q_scale, unit_eps;
  const float* pre; long long ld_pre;       // register form only: fp32 rows [k unit | q unit * q_scale | decay | v | sigmoid(beta)] (delta_prepare_kernel)
};

// Operands of `nt` tokens (rows t0 ..) of head h for a delta-rule CTA: kq[jj] = [k unit | q unit * q_scale | decay], each `ldn` >= N
// floats wide (zeros behind N), vs[jj] = the CTA's PB value columns (zeros behind the head's last column), bs[jj] = sigmoid(beta).
// All threads load element-wise (independent loads), then one warp per token takes the two sums of squares from shared memory and
// rescales.  Ends with a barrier.
template <typename AT>
__device__ __forceinline__ void delta_stage(const DeltaArgs& a, long long t0, int nt, int h, int g, int p0, int PB, float negA, float* kq, float* vs,
                                            float* bs, int ldn) {
  const int N = a.N, GN = a.G * N, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const AT* in = reinterpret_cast<const AT*>(a.in);
#pragma unroll 4
  for (int e = threadIdx.x; e < nt * ldn; e += blockDim.x) {
    const int jj = e / ldn, n = e - jj * ldn;
    float* dst = kq + jj * 3 * ldn;
    float kv = 0.f, qv = 0.f, gv = 0.f;
    if (n < N) {
      const AT* row = in + (t0 + jj) * a.ld_in;
      kv = ldf<AT>(row + GN + g * N + n);
      qv = ldf<AT>(row + g * N + n);
      gv = expf(negA * softplus_f(a.dt[(t0 + jj) * a.ld_dt + h * N + n] + a.dt_bias[h * N + n]));
    }
    dst[n] = kv; dst[ldn + n] = qv; dst[2 * ldn + n] = gv;
  }
#pragma unroll 2
  for (int e = threadIdx.x; e < nt * PB; e += blockDim.x) {
    const int jj = e / PB, c = e - jj * PB;
    vs[e] = p0 + c < a.P ? ldf<AT>(in + (t0 + jj) * a.ld_in + 2 * GN + h * a.P + p0 + c) : 0.f;
  }
  if (threadIdx.x < nt) bs[threadIdx.x] = sigmoid_f(ldf<AT>((const AT*)a.beta + (t0 + threadIdx.x) * a.ld_b + h));
  __syncthreads();
  for (int jj = warp; jj < nt; jj += nw) {
    float* dst = kq + jj * 3 * ldn;
    float sk = 0.f, sq = 0.f;
    for (int n = lane; n < N; n += 32) { sk += dst[n] * dst[n]; sq += dst[ldn + n] * dst[ldn + n]; }
    const float ik = 1.f / sqrtf(warp_sum(sk) + a.unit_eps), iq = a.q_scale / sqrtf(warp_sum(sq) + a.unit_eps);
    for (int n = lane; n < N; n += 32) { dst[n] *= ik; dst[ldn + n] *= iq; }
  }
  __syncthreads();
}

// The token-wise part of the delta rule's operands, once per step instead of once per column block, as fp32 rows
// [k unit: G N | q unit * q_scale: G N | decay: H N | v: H P | sigmoid(beta): H] (row stride ld_pre, a multiple of 4 floats), so that
// the scan can fetch them with asynchronous copies.                                                          grid (T), block 256
__host__ __device__ inline long long delta_pre_width(int G, int H, int N, int P) { return ((long long)(2 * G + H) * N + (long long)H * P + H + 3) / 4 * 4; }

template <typename AT>
__global__ void delta_prepare_kernel(DeltaArgs a, float* __restrict__ pre) {
  const long long t = blockIdx.x;
  const int N = a.N, GN = a.G * N, HN = a.H * N, HP = a.H * a.P, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const AT* row = reinterpret_cast<const AT*>(a.in) + t * a.ld_in;
  float* out = pre + t * a.ld_pre;
  for (int gi = warp; gi < a.G; gi += nw) {
    float sk = 0.f, sq = 0.f;
    for (int n = lane; n < N; n += 32) {
      const float qv = ldf<AT>(row + gi * N + n), kv = ldf<AT>(row + GN + gi * N + n);
      sk += kv * kv; sq += qv * qv;
    }
    const float ik = 1.f / sqrtf(warp_sum(sk) + a.unit_eps), iq = a.q_scale / sqrtf(warp_sum(sq) + a.unit_eps);
    for (int n = lane; n < N; n += 32) {
      out[gi * N + n] = ldf<AT>(row + GN + gi * N + n) * ik;
      out[GN + gi * N + n] = ldf<AT>(row + gi * N + n) * iq;
    }
  }
  for (int e = threadIdx.x; e < HN; e += blockDim.x)
    out[2 * GN + e] = expf(-expf(a.A_log[e / N]) * softplus_f(a.dt[t * a.ld_dt + e] + a.dt_bias[e]));
  for (int e = threadIdx.x; e < HP; e += blockDim.x) out[2 * GN + HN + e] = ldf<AT>(row + 2 * GN + e);
  for (int e = threadIdx.x; e < a.H; e += blockDim.x) out[2 * GN + HN + HP + e] = sigmoid_f(ldf<AT>((const AT*)a.beta + t * a.ld_b + e));
}

__device__ __forceinline__ void cp_async_16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

constexpr int kDeltaTokensMax = 16;

// One CTA per (sequence, head, block of PB value columns): the columns of S evolve independently.  S[N][PB] in shared memory; thread
// (r, p) owns rows n = r, r + R, .. of column p.  Per block of tokens the operands are staged by one warp per token (unit vectors of
// q and k by a warp reduction, decays and the write strength in fp32); per token two barriers:
//   S <- g S, partial S^T k  |  u = beta (v - S^T k), S <- S + k u^T, partial S^T q  |  o
template <typename AT>
__global__ void delta_scan_kernel(DeltaArgs a, int PB, int R, int kTok) {
  extern __shared__ __align__(16) float smem[];
  const int b = blockIdx.x, h = blockIdx.y, N = a.N, P = a.P, H = a.H, p0 = blockIdx.z * PB;
  const int g = h / (H / a.G);
  const bool vec4 = PB % 4 == 0 && P % 4 == 0;          // 16-byte copies of the state block (rows of PB floats at a stride of P)
  const int p = threadIdx.x % PB, r = threadIdx.x / PB, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  float* S = smem;                          // [N][PB]
  float* red1 = S + N * PB;                 // [R][PB]
  float* red2 = red1 + R * PB;              // [R][PB]
  float* kq = red2 + R * PB;                // [tokens][3N]   k | q | g
  float* vs = kq + kTok * 3 * N;            // [tokens][PB]
  float* bs = vs + kTok * PB;               // [tokens]
  const int s = a.cu[b], q = a.cu[b + 1] - s;
  if (q == 0) return;
  const bool fresh = a.ctx[b] - q == 0;
  float* gS = a.state + ((long long)a.slots[b] * H + h) * N * P;
  if (vec4) {
    for (int e = 4 * threadIdx.x; e < N * PB; e += 4 * blockDim.x) {
      const int n = e / PB, c = e % PB;
      *reinterpret_cast<float4*>(S + e) = fresh ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(gS + n * P + p0 + c);
    }
  } else {
    for (int e = threadIdx.x; e < N * PB; e += blockDim.x) { const int n = e / PB, c = e % PB; S[e] = fresh ? 0.f : gS[n * P + p0 + c]; }
  }
  const AT* in = reinterpret_cast<const AT*>(a.in);
  const float negA = -expf(a.A_log[h]);
  const int GN = a.G * N;
  for (int j0 = 0; j0 < q; j0 += kTok) {
    const int nt = min(kTok, q - j0);
    __syncthreads();                        // the last block's operands are no longer read (and the state is loaded)
    delta_stage<AT>(a, s + j0, nt, h, g, p0, PB, negA, kq, vs, bs, N);
    for (int jj = 0; jj < nt; ++jj) {
      const float* kr = kq + jj * 3 * N;
      if (r < R) {
        float acc = 0.f;
        for (int n = r; n < N; n += R) {
          const float sv = kr[2 * N + n] * S[n * PB + p];
          S[n * PB + p] = sv;
          acc += sv * kr[n];
        }
        red1[r * PB + p] = acc;
      }
      __syncthreads();
      if (r < R) {
        float sk = 0.f;
        for (int i = 0; i < R; ++i) sk += red1[i * PB + p];
        const float u = bs[jj] * (vs[jj * PB + p] - sk);
        float acc = 0.f;
        for (int n = r; n < N; n += R) {
          const float sv = S[n * PB + p] + kr[n] * u;
          S[n * PB + p] = sv;
          acc += sv * kr[N + n];
        }
        red2[r * PB + p] = acc;
      }
      __syncthreads();
      if (r == 0) {
        float y = 0.f;
        for (int i = 0; i < R; ++i) y += red2[i * PB + p];
        a.out[(long long)(s + j0 + jj) * H * P + h * P + p0 + p] = y;
      }
    }
  }
  __syncthreads();
  if (vec4) {
    for (int e = 4 * threadIdx.x; e < N * PB; e += 4 * blockDim.x) {
      const int n = e / PB, c = e % PB;
      *reinterpret_cast<float4*>(gS + n * P + p0 + c) = *reinterpret_cast<const float4*>(S + e);
    }
  } else {
    for (int e = threadIdx.x; e < N * PB; e += blockDim.x) { const int n = e / PB, c = e % PB; gS[n * P + p0 + c] = S[e]; }
  }
}

// The same recurrence with the state in REGISTERS, for portions of many tokens (bound by the latency of a token, not by the state's
// bytes): L lanes share a value column, lane l holding the key rows 4 (l + L j) + e (j < NR4, e < 4: 16-byte shared-memory loads of k, q
// and the decay, consecutive over the lanes), so a warp runs 32 / L columns at once, both products S^T k and S^T q end in log2(L)
// shuffles, and a token needs no block barrier.  The operands of 16 tokens at a time come from delta_prepare_kernel's rows by asynchronous
// copies into one of two buffers while the block before is computed (rows padded with zeros to 4 L NR4, so the token loop has no
// bounds checks).                                                                grid (B, H, ceil(P / PB)), PB = warps * 32 / L
constexpr int kDeltaWarpMinTokens = 8;      // shorter steps are bound by the state copies: the shared-memory kernel with 16-byte copies runs

template <typename AT, int L, int NR4>
__global__ void delta_scan_warp_kernel(DeltaArgs a, int kTok) {
  constexpr int CPW = 32 / L, NP = 4 * L * NR4;
  extern __shared__ __align__(16) float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, PB = nw * CPW;
  const int l = lane % L, cw = lane / L;
  const int b = blockIdx.x, h = blockIdx.y, N = a.N, P = a.P, H = a.H, p0 = blockIdx.z * PB;
  const int g = h / (H / a.G), col = warp * CPW + cw, pc = p0 + col;
  const bool colok = pc < P;
  const int per = 3 * NP + PB + 4;          // floats of one token: k | q | g | v | beta (padded to 16 bytes)
  const int s = a.cu[b], q = a.cu[b + 1] - s;
  if (q == 0) return;
  const bool fresh = a.ctx[b] - q == 0;
  float* gS = a.state + ((long long)a.slots[b] * H + h) * N * P;
  float st[4 * NR4];
#pragma unroll
  for (int j = 0; j < NR4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = 4 * (l + L * j) + e;
      st[4 * j + e] = (!fresh && colok && n < N) ? gS[(long long)n * P + pc] : 0.f;
    }
  // both staging buffers start as zeros: rows behind N and columns behind P are never copied
  for (int e = threadIdx.x; e < 2 * kTok * per; e += blockDim.x) smem[e] = 0.f;
  __syncthreads();
  const int GN = a.G * N, HN = H * N, vw = min(PB, P - p0);
  const bool vec = N % 4 == 0 && P % 4 == 0 && PB % 4 == 0;          // 16-byte copies: every segment starts and ends on a 16-byte boundary
  const int n4 = vec ? N / 4 : N, v4 = vec ? vw / 4 : vw, items = 3 * n4 + v4 + 1;
  // asynchronous copies of the operands of tokens t0 .. t0 + nt into buffer `buf`: all of a block are in flight at once
  auto fetch = [&](long long t0, int nt, float* buf) {
    for (int e = threadIdx.x; e < nt * items; e += blockDim.x) {
      const int jj = e / items, c = e - jj * items;
      const float* pr = a.pre + (t0 + jj) * a.ld_pre;
      float* dst = buf + jj * per;
      if (c >= 3 * n4 + v4) { cp_async_4(dst + 3 * NP + PB, pr + 2 * GN + HN + H * P + h); continue; }
      const int seg = c < 3 * n4 ? c / n4 : 3, i = c - seg * n4;
      const float* src = seg == 0 ? pr + g * N : seg == 1 ? pr + GN + g * N : seg == 2 ? pr + 2 * GN + h * N : pr + 2 * GN + HN + h * P + p0;
      float* d = seg == 3 ? dst + 3 * NP : dst + seg * NP;
      if (vec) cp_async_16(d + 4 * i, src + 4 * i); else cp_async_4(d + i, src + i);
    }
    cp_async_commit();
  };
  fetch(s, min(kTok, q), smem);
  int blk = 0;
  for (int j0 = 0; j0 < q; j0 += kTok, ++blk) {
    const int nt = min(kTok, q - j0);
    cp_async_wait_all();
    __syncthreads();                        // this block's operands have landed for every thread; the other buffer is no longer read
    if (j0 + kTok < q) fetch(s + j0 + kTok, min(kTok, q - j0 - kTok), smem + ((blk + 1) & 1) * kTok * per);
    const float* cur = smem + (blk & 1) * kTok * per;
    for (int jj = 0; jj < nt; ++jj) {
      const float* tk = cur + jj * per;
      const float4* k4 = reinterpret_cast<const float4*>(tk) + l;
      const float4* q4 = k4 + NP / 4;
      const float4* g4 = k4 + 2 * (NP / 4);
      float a0 = 0.f, a1 = 0.f;
#pragma unroll
      for (int j = 0; j < NR4; ++j) {
        const float4 kk = k4[j * L], gg = g4[j * L];
        st[4 * j] *= gg.x; st[4 * j + 1] *= gg.y; st[4 * j + 2] *= gg.z; st[4 * j + 3] *= gg.w;
        a0 += st[4 * j] * kk.x + st[4 * j + 2] * kk.z;
        a1 += st[4 * j + 1] * kk.y + st[4 * j + 3] * kk.w;
      }
      float sk = a0 + a1;
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) sk += __shfl_xor_sync(0xffffffffu, sk, o);
      const float u = tk[3 * NP + PB] * (tk[3 * NP + col] - sk);
      a0 = 0.f; a1 = 0.f;
#pragma unroll
      for (int j = 0; j < NR4; ++j) {
        const float4 kk = k4[j * L], qq = q4[j * L];
        st[4 * j] += kk.x * u; st[4 * j + 1] += kk.y * u; st[4 * j + 2] += kk.z * u; st[4 * j + 3] += kk.w * u;
        a0 += st[4 * j] * qq.x + st[4 * j + 2] * qq.z;
        a1 += st[4 * j + 1] * qq.y + st[4 * j + 3] * qq.w;
      }
      float y = a0 + a1;
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (l == 0 && colok) a.out[(long long)(s + j0 + jj) * H * P + h * P + pc] = y;
    }
  }
#pragma unroll
  for (int j = 0; j < NR4; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int n = 4 * (l + L * j) + e;
      if (colok && n < N) gS[(long long)n * P + pc] = st[4 * j + e];
    }
}

// ---------------------------------------------------------------------------------------------------------- minGRU
// z = sigmoid(rows[z]), c = u + 1/2 (u >= 0) or sigmoid(u), S <- (1 - z) S + z c, out = S * silu(rows[g]) * out_mult.
// The recurrence is linear in S, so a sequence's tokens are cut into TS slices: thread (channel, slice) first folds its slice into
// (A, B) with S_end = A S_start + B, then takes its start from the slices before it (at most TS - 1 steps) and runs its slice again,
// writing the outputs.  Decode (one token) is the TS = 1 case.                     grid (B, ceil(R / 32)), block (32 channels, TS)
template <typename AT>
__global__ void mingru_scan_kernel(const AT* __restrict__ rows, long long ld, int z0, int x0, int g0, int R, float* __restrict__ state,
                                   const int* __restrict__ cu, const int* __restrict__ ctx, const int* __restrict__ slots, float out_mult,
                                   AT* __restrict__ out, long long ld_out) {
  __shared__ float fa[32][33], fb[32][33];
  const int b = blockIdx.x, cl = threadIdx.x, sl = threadIdx.y, TS = blockDim.y, c = blockIdx.y * 32 + cl;
  const int s = cu[b], q = cu[b + 1] - s;
  if (q == 0) return;
  const int len = (q + TS - 1) / TS, j0 = min(q, sl * len), j1 = min(q, j0 + len);
  const bool live = c < R;
  const AT* row = rows + (long long)(s + j0) * ld + c;
  float A = 1.f, Bv = 0.f;
  if (live && TS > 1) {
    const AT* r = row;
#pragma unroll 4
    for (int j = j0; j < j1; ++j, r += ld) {
      const float z = sigmoid_f(ldf<AT>(r + z0)), u = ldf<AT>(r + x0);
      const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
      A *= 1.f - z;
      Bv = (1.f - z) * Bv + z * cand;
    }
  }
  fa[sl][cl] = A; fb[sl][cl] = Bv;
  __syncthreads();
  if (!live) return;
  float* st = state + (long long)slots[b] * R + c;
  float S = ctx[b] - q == 0 ? 0.f : *st;
  for (int i = 0; i < sl; ++i) S = fa[i][cl] * S + fb[i][cl];
  AT* orow = out + (long long)(s + j0) * ld_out + c;
#pragma unroll 4
  for (int j = j0; j < j1; ++j, row += ld, orow += ld_out) {
    const float z = sigmoid_f(ldf<AT>(row + z0)), u = ldf<AT>(row + x0), gr = ldf<AT>(row + g0);
    const float cand = u >= 0.f ? u + 0.5f : sigmoid_f(u);
    S = (1.f - z) * S + z * cand;
    stf<AT>(orow, S * silu_f(gr) * out_mult);
  }
  if (sl == TS - 1) *st = S;          // the last slice ends at the sequence's last token (empty slices pass S through)
}

// ---------------------------------------------------------------------------------------------------------- attention prologue
// One warp per head of a token (query heads first, then key heads): x / sqrt(mean(x^2) + eps) * w, then adjacent pairs (2i, 2i+1) of the
// first `rot` entries turn by pos * inv_freq[i].  Queries -> qout fp32 [T, H, D]; keys and the untouched values -> the paged pools.
template <typename AT>
__global__ void qk_norm_rope_append_kernel(const AT* __restrict__ rows, long long ld, int q0, int k0, int v0, int H, int G, int D, int V,
                                           const float* __restrict__ qn, const float* __restrict__ kn, float eps,
                                           const float* __restrict__ inv_freq, int rot, const int* __restrict__ positions,
                                           const int* __restrict__ slot_map, int page, float* __restrict__ qout, AT* __restrict__ kpool,
                                           AT* __restrict__ vpool) {
  const long long t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const float pos = (float)positions[t];
  const int slot = slot_map[t], pg = slot / page, off = slot % page;
  const AT* r = rows + t * ld;
  for (int hh = warp; hh < H + G; hh += nw) {
    const bool isq = hh < H;
    const AT* src = isq ? r + q0 + hh * D : r + k0 + (hh - H) * D;
    const float* w = isq ? qn : kn;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) { const float v = ldf<AT>(src + d); ss += v * v; }
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)D + eps);
    float* qd = qout + (t * H + hh) * D;
    AT* kd = kpool + (((long long)pg * G + (hh - H)) * page + off) * D;
    for (int d0 = 0; d0 < D; d0 += 32) {        // all lanes take part in the shuffle; d even <-> lane even
      const int d = d0 + lane;
      float v = d < D ? ldf<AT>(src + d) * inv * w[d] : 0.f;
      const float other = __shfl_xor_sync(0xffffffffu, v, 1);
      if (d < rot) {
        float sn, cs;
        sincosf(pos * inv_freq[d >> 1], &sn, &cs);
        v = (d & 1) ? v * cs + other * sn : v * cs - other * sn;
      }
      if (d < D) { if (isq) qd[d] = v; else stf<AT>(kd + d, v); }
    }
  }
  for (int i = threadIdx.x; i < G * V; i += blockDim.x) vpool[(((long long)pg * G + i / V) * page + off) * V + i % V] = r[v0 + i];
}

// ---------------------------------------------------------------------------------------------------------- attention with a sink
struct SinkAttnArgs {
  const float* q;                           // fp32 [T, H, D] (normed, rotated)
  const void* kpool; const void* vpool;     // [pages, G, page, D] / [pages, G, page, V]
  const float* sink;                        // [H] (nullable)
  const int* block_tables; int max_blocks;
  const int* positions; const int* cu; int B;
  int H, G, D, V, page;
  int block, window;                        // visible keys j <= p: same block of `block` positions (0: all), p - j < window (0: all)
  float scale, out_mult;
  void* out; long long ld_out;              // AT, row t at out + t * ld_out, head h at column h * V
  int nsplit, chunk;
  float* part;                              // [T, H, nsplit, V + 2] = (m, l, o[V]) when the keys are split
};

constexpr int kTile = 32;

__device__ __forceinline__ int first_key(int pos, int block, int window) {
  int lo = block > 0 ? pos / block * block : 0;
  if (window > 0) lo = max(lo, pos - window + 1);
  return lo;
}

// value column of register i of a lane: VEC (vdim a multiple of 128) 4 lane + 128 (i / 4) + i % 4 — four adjacent columns per 16-byte
// shared-memory load —, else lane + 32 i
template <bool VEC>
__device__ __forceinline__ int sink_vcol(int lane, int i) { return VEC ? 4 * lane + 128 * (i >> 2) + (i & 3) : lane + 32 * i; }

// grid (tokens, G * ceil((H/G) / warps), key splits); one warp per query head, the warps of a CTA share one key / value head whose tile
// of kTile keys and values is staged in shared memory as floats.  Lane j scores key j of the tile; the running softmax (m, l) and the
// accumulator live in registers, lane owning the value columns sink_vcol(lane, i).  Key splits count from the first visible key.
// VEC (dim a multiple of the 16-byte chunk, vdim a multiple of 128): 16-byte shared-memory stores and loads in all phases, key rows
// padded by 4 floats; else scalar accesses, key rows padded by 1.
template <typename AT, int NPL, bool VEC>
__global__ void sink_attention_kernel(SinkAttnArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D = a.D, V = a.V, ldk = VEC ? D + 4 : D + 1;
  float* qs = smem;                         // [nw][D]
  float* ks = qs + nw * D;                  // [tile][D + 1]
  float* vs = ks + kTile * ldk;             // [tile][V]
  const int t = blockIdx.x, Rg = a.H / a.G, nb = (Rg + nw - 1) / nw;
  const int g = blockIdx.y / nb, r = (blockIdx.y % nb) * nw + warp, h = g * Rg + r;
  const bool valid = r < Rg;
  const int pos = a.positions[t];
  const int* bt = a.block_tables + (long long)seq_of(a.cu, a.B, t) * a.max_blocks;
  for (int i = threadIdx.x; i < nw * D; i += blockDim.x) {
    const int rr = (blockIdx.y % nb) * nw + i / D;
    qs[i] = rr < Rg ? a.q[((long long)t * a.H + g * Rg + rr) * D + i % D] * a.scale : 0.f;
  }
  float m = -INFINITY, l = 0.f, o[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) o[i] = 0.f;
  const float* qh = qs + warp * D;
  const int lo = first_key(pos, a.block, a.window);
  const long long jb = (long long)lo + (long long)blockIdx.z * a.chunk;
  const int jbeg = (int)min(jb, (long long)pos + 1), jend = (int)min((long long)pos + 1, jb + a.chunk);
  constexpr int E = 16 / (int)sizeof(AT);
  const bool vec = D % E == 0 && V % E == 0;
  for (int j0 = jbeg; j0 < jend; j0 += kTile) {
    __syncthreads();
    const int nk = min(kTile, jend - j0);
    for (int jj = warp; jj < nk; jj += nw) {            // each warp fetches whole rows: one block-table lookup per row
      const int j = j0 + jj;
      const long long base = ((long long)bt[j / a.page] * a.G + g) * a.page + j % a.page;
      const AT* ksrc = (const AT*)a.kpool + base * D;
      const AT* vsrc = (const AT*)a.vpool + base * V;
      float* kd = ks + jj * ldk;
      float* vd = vs + jj * V;
      if (VEC) {
        for (int c = lane; c < (D + V) / E; c += 32) {
          float f[E];
          unpack16<AT>(*reinterpret_cast<const uint4*>(c < D / E ? ksrc + c * E : vsrc + (c - D / E) * E), f);
          float* dst = c < D / E ? kd + c * E : vd + (c - D / E) * E;
#pragma unroll
          for (int e = 0; e < E; e += 4) *reinterpret_cast<float4*>(dst + e) = make_float4(f[e], f[e + 1], f[e + 2], f[e + 3]);
        }
      } else if (vec) {
        for (int c = lane; c < D / E; c += 32) { float f[E]; unpack16<AT>(*reinterpret_cast<const uint4*>(ksrc + c * E), f);
#pragma unroll
          for (int e = 0; e < E; ++e) kd[c * E + e] = f[e]; }
        for (int c = lane; c < V / E; c += 32) unpack16<AT>(*reinterpret_cast<const uint4*>(vsrc + c * E), vd + c * E);
      } else {
        for (int d = lane; d < D; d += 32) kd[d] = ldf<AT>(ksrc + d);
        for (int d = lane; d < V; d += 32) vd[d] = ldf<AT>(vsrc + d);
      }
    }
    __syncthreads();
    if (!valid) continue;
    float sc = -INFINITY;
    if (lane < nk) {
      const float* kr = ks + lane * ldk;
      float d = 0.f;
      if (VEC) {
        const float4* q4 = reinterpret_cast<const float4*>(qh);
        const float4* k4 = reinterpret_cast<const float4*>(kr);
        for (int i = 0; i < (D >> 2); ++i) { const float4 x = q4[i], y = k4[i]; d += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w; }
      } else {
        for (int i = 0; i < D; ++i) d += qh[i] * kr[i];
      }
      sc = d;
    }
    const float nm = fmaxf(m, warp_max(sc));
    const float cf = m == -INFINITY ? 0.f : expf(m - nm);
    const float pw = lane < nk ? expf(sc - nm) : 0.f;
    l = l * cf + warp_sum(pw);
    m = nm;
#pragma unroll
    for (int i = 0; i < NPL; ++i) o[i] *= cf;
    for (int jj = 0; jj < nk; ++jj) {
      const float w = __shfl_sync(0xffffffffu, pw, jj);
      const float* vr = vs + jj * V;
      if (VEC) {
#pragma unroll
        for (int i = 0; i < NPL / 4; ++i)
          if (128 * i < V) {
            const float4 c = *reinterpret_cast<const float4*>(vr + 4 * lane + 128 * i);
            o[4 * i] += w * c.x; o[4 * i + 1] += w * c.y; o[4 * i + 2] += w * c.z; o[4 * i + 3] += w * c.w;
          }
      } else {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          const int d = lane + 32 * i;
          if (d < V) o[i] += w * vr[d];
        }
      }
    }
  }
  if (!valid) return;
  if (a.nsplit == 1) {
    // the query's own position is always visible: l > 0.  The sink joins the denominator only: exp(sink - m), no value.
    if (a.sink != nullptr) l += expf(a.sink[h] - m);
    const float inv = a.out_mult / l;
    AT* orow = (AT*)a.out + (long long)t * a.ld_out + (long long)h * V;
#pragma unroll
    for (int i = 0; i < NPL; ++i) { const int d = sink_vcol<VEC>(lane, i); if (d < V) stf<AT>(orow + d, o[i] * inv); }
  } else {
    float* pp = a.part + (((long long)t * a.H + h) * a.nsplit + blockIdx.z) * (V + 2);
    if (lane == 0) { pp[0] = m; pp[1] = l; }
#pragma unroll
    for (int i = 0; i < NPL; ++i) { const int d = sink_vcol<VEC>(lane, i); if (d < V) pp[2 + d] = o[i]; }
  }
}

// merge the key splits of one (token, head): o = sum_z o_z e^(m_z - M) / (sum_z l_z e^(m_z - M) + e^(sink - M)).  One warp each.
template <typename AT, int NPL>
__global__ void sink_combine_kernel(const float* __restrict__ part, const float* __restrict__ sink, int H, int V, int nsplit, float out_mult,
                                    AT* __restrict__ out, long long ld_out) {
  const long long th = blockIdx.x;
  const int lane = threadIdx.x, h = (int)(th % H);
  const float* pp = part + th * nsplit * (V + 2);
  float M = -INFINITY, den = 0.f, acc[NPL];
  for (int z = 0; z < nsplit; ++z) M = fmaxf(M, pp[(long long)z * (V + 2)]);
#pragma unroll
  for (int i = 0; i < NPL; ++i) acc[i] = 0.f;
  for (int z = 0; z < nsplit; ++z) {
    const float* pz = pp + (long long)z * (V + 2);
    if (pz[0] == -INFINITY) continue;                 // a split beyond this token's keys
    const float e = expf(pz[0] - M);
    den += pz[1] * e;
#pragma unroll
    for (int i = 0; i < NPL; ++i) { const int d = lane + 32 * i; if (d < V) acc[i] += pz[2 + d] * e; }
  }
  if (sink != nullptr) den += expf(sink[h] - M);
  const float inv = out_mult / den;
  AT* orow = out + (th / H) * ld_out + (long long)h * V;
#pragma unroll
  for (int i = 0; i < NPL; ++i) { const int d = lane + 32 * i; if (d < V) stf<AT>(orow + d, acc[i] * inv); }
}

// ---------------------------------------------------------------------------------------------------------- router
// One warp per token.  s = softmax(z) over all E experts; choice c = s + corr; groups = ng equal runs of neighbours, a group's value is
// its largest c; experts outside the `keep` best groups count as -inf; the `top` largest c win (ties: lowest id); weights = their s.
__global__ void group_softmax_topk_kernel(const float* __restrict__ z, long long ld_z, const float* __restrict__ corr, int E, int top, int ng, int keep,
                                          int* __restrict__ idx, float* __restrict__ w) {
  extern __shared__ float sh[];
  float* sc = sh;                            // [E] plain scores
  float* ch = sh + E;                        // [E] choice scores
  float* gv = ch + E;                        // [ng]
  const long long t = blockIdx.x;
  const int lane = threadIdx.x;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[t * ld_z + e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) { const float v = expf(z[t * ld_z + e] - mx); sc[e] = v; sum += v; }
  sum = warp_sum(sum);
  for (int e = lane; e < E; e += 32) { const float s = sc[e] / sum; sc[e] = s; ch[e] = s + (corr != nullptr ? corr[e] : 0.f); }
  __syncwarp();
  if (ng > 1 && keep < ng) {
    const int per = E / ng;
    for (int gi = lane; gi < ng; gi += 32) {
      float b = -INFINITY;
      for (int e = gi * per; e < (gi + 1) * per; ++e) b = fmaxf(b, ch[e]);
      gv[gi] = b;
    }
    __syncwarp();
    // drop the ng - keep worst groups: repeatedly the smallest value, ties to the HIGHEST id (so that kept ties go to the lowest)
    for (int j = 0; j < ng - keep; ++j) {
      float worst = INFINITY; int wi = -1;
      for (int gi = lane; gi < ng; gi += 32) { const float v = gv[gi]; if (v <= worst) { worst = v; wi = gi; } }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, worst, o);
        const int oi = __shfl_xor_sync(0xffffffffu, wi, o);
        if (oi >= 0 && (wi < 0 || ov < worst || (ov == worst && oi > wi))) { worst = ov; wi = oi; }
      }
      if (lane == 0) gv[wi] = INFINITY;      // marked as dropped
      __syncwarp();
      for (int e = wi * per + lane; e < (wi + 1) * per; e += 32) ch[e] = -INFINITY;
      __syncwarp();
    }
  }
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) { const float v = ch[e]; if (v > best) { best = v; bi = e; } }   // ascending e: first maximum wins
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { idx[t * top + j] = bi; w[t * top + j] = sc[bi]; ch[bi] = -INFINITY; }
    __syncwarp();
  }
}

}  // namespace

// =========================================================================================================== launchers
cudaError_t stream_embed_launch(const void* table, bool table_f32, long long ld, const long long* ids, float scale, int S, int n, float* xs, int T,
                                cudaStream_t s) {
  if (S < 1 || S > kMaxStreams) return cudaErrorInvalidValue;
  dim3 grid(T, (n + 1023) / 1024);
  if (table_f32) stream_embed_kernel<float><<<grid, 256, 0, s>>>((const float*)table, ld, ids, scale, S, n, xs);
  else stream_embed_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)table, ld, ids, scale, S, n, xs);
  return last();
}

cudaError_t hyper_step_launch(float* xs, const float* y, long long ld_y, const float* y2, long long ld_y2, const void* gate, long long ld_g,
                              const float* ls, const float* mix, const float* out_w, float mult, const float* in_w, float alpha, const float* w,
                              const float* b, void* xa, bool f32, int S, int n, int T, cudaStream_t s) {
  if (S < 1 || S > kMaxStreams) return cudaErrorInvalidValue;
  HyperArgs a{xs, y, ld_y, y2, ld_y2, gate, ld_g, ls, mix, out_w, in_w, w, b, mult, alpha, xa, S, n};
  dim3 grid(T, (n + 255) / 256);
  AT_DISPATCH(f32, (hyper_step_kernel<AT><<<grid, 256, 0, s>>>(a)));
  return last();
}

cudaError_t relu2_launch(void* x, long long ld, int n, bool f32, int T, cudaStream_t s) {
  dim3 grid(T, (n + 1023) / 1024);
  AT_DISPATCH(f32, (relu2_kernel<AT><<<grid, 256, 0, s>>>((AT*)x, ld, n)));
  return last();
}

cudaError_t delta_scan_launch(const void* in, long long ld_in, const void* beta, long long ld_b, const float* dt, long long ld_dt,
                              const float* dt_bias, const float* A_log, float* state, const int* cu, const int* ctx, const int* slots, float* out,
                              int B, int H, int G, int N, int P, float q_scale, float unit_eps, bool f32, int max_q, float* pre, int T, cudaStream_t s) {
  if (G < 1 || H % G != 0 || P < 1 || N < 1) return cudaErrorInvalidValue;
  DeltaArgs a{in, ld_in, beta, ld_b, dt, ld_dt, dt_bias, A_log, state, cu, ctx, slots, out, H, G, N, P, q_scale, unit_eps, nullptr, 0};
  if (delta_scan_wants_prepare(N, max_q)) {
    if (pre == nullptr) return cudaErrorInvalidValue;
    a.pre = pre; a.ld_pre = delta_pre_width(G, H, N, P);
    AT_DISPATCH(f32, (delta_prepare_kernel<AT><<<T, 256, 0, s>>>(a, pre)));
    // register form: 4 lanes per value column (8 beyond 128 key rows), up to 4 warps per CTA.  A warp's time per token is its serial
    // instruction count, so while the grid leaves SMs idle (one short batch) a column is spread over more lanes: fewer rows per lane,
    // one more shuffle level, twice the CTAs
    int L = N <= 128 ? 4 : 8;
    auto ctas = [&](int lanes) { const int pb = 4 * (32 / lanes); return (long long)B * H * ((P + pb - 1) / pb); };
    while (L < 16 && ctas(L) < 148 && N > 4 * L) L *= 2;
    const int cpw = 32 / L;
    const int need = (N + 4 * L - 1) / (4 * L), nr4 = need <= 1 ? 1 : need <= 2 ? 2 : need <= 4 ? 4 : 8;
    int nwarps = (P + cpw - 1) / cpw;
    if (nwarps > 4) nwarps = 4;
    const int PB = nwarps * cpw, NP = 4 * L * nr4;
    const int stage = max_q < kDeltaTokensMax ? max_q : kDeltaTokensMax;
    const size_t smem = 2 * (size_t)stage * (3 * NP + PB + 4) * sizeof(float);
    auto go = [&](auto k) -> cudaError_t {
      if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
      k<<<dim3(B, H, (P + PB - 1) / PB), 32 * nwarps, smem, s>>>(a, stage);
      return last();
    };
#define DELTA_CASE(LL, R) if (L == LL && nr4 == R) { AT_DISPATCH(f32, return go(delta_scan_warp_kernel<AT, LL, R>)); }
    DELTA_CASE(4, 1) DELTA_CASE(4, 2) DELTA_CASE(4, 4) DELTA_CASE(4, 8)
    DELTA_CASE(8, 1) DELTA_CASE(8, 2) DELTA_CASE(8, 4) DELTA_CASE(8, 8)
    DELTA_CASE(16, 1) DELTA_CASE(16, 2) DELTA_CASE(16, 4)
#undef DELTA_CASE
    return cudaErrorInvalidValue;
  }
  // columns of the state are independent: split a head's value dimension over CTAs (PB columns each) while the grid is small
  int PB = P;
  while (PB > 16 && PB % 2 == 0 && ((long long)B * H * (P / PB) < 592 || PB > 256)) PB /= 2;
  if (PB > 1024) return cudaErrorInvalidValue;
  int R = 256 / PB;
  if (R < 1) R = 1;
  if (R > N) R = N;
  const int threads = (R * PB + 31) / 32 * 32;   // tail threads (r >= R) only help with staging and the state copy
  int stage = max_q < 1 ? 1 : (max_q < kDeltaTokensMax ? max_q : kDeltaTokensMax);
  auto bytes = [&](int st) { return ((size_t)N * PB + 2 * (size_t)R * PB + (size_t)st * (3 * N + PB + 1)) * sizeof(float); };
  while (stage > 1 && bytes(stage) > 200 * 1024) stage /= 2;
  const size_t smem = bytes(stage);
  if (smem > 220 * 1024) return cudaErrorInvalidValue;
  if (f32) {
    auto k = delta_scan_kernel<float>;
    if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
    k<<<dim3(B, H, P / PB), threads, smem, s>>>(a, PB, R, stage);
  } else {
    auto k = delta_scan_kernel<__nv_bfloat16>;
    if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
    k<<<dim3(B, H, P / PB), threads, smem, s>>>(a, PB, R, stage);
  }
  return last();
}

cudaError_t mingru_scan_launch(const void* rows, long long ld, int z0, int x0, int g0, int R, float* state, const int* cu, const int* ctx,
                               const int* slots, float out_mult, void* out, long long ld_out, int B, bool f32, int max_q, cudaStream_t s) {
  int TS = 1;                                   // slices of at least 16 tokens, at most 32 of them
  while (TS < 32 && max_q >= 32 * TS) TS *= 2;
  dim3 grid(B, (R + 31) / 32), block(32, TS);
  AT_DISPATCH(f32, (mingru_scan_kernel<AT><<<grid, block, 0, s>>>((const AT*)rows, ld, z0, x0, g0, R, state, cu, ctx, slots, out_mult, (AT*)out, ld_out)));
  return last();
}

cudaError_t qk_norm_rope_append_launch(const void* rows, long long ld, int q0, int k0, int v0, int H, int G, int D, int V, const float* qn,
                                       const float* kn, float eps, const float* inv_freq, int rot, const int* positions, const int* slot_map,
                                       int page, float* qout, void* kpool, void* vpool, bool f32, int T, cudaStream_t s) {
  if (rot % 2 != 0 || rot > D) return cudaErrorInvalidValue;
  const int threads = 32 * (H + G < 8 ? H + G : 8);
  AT_DISPATCH(f32, (qk_norm_rope_append_kernel<AT><<<T, threads, 0, s>>>((const AT*)rows, ld, q0, k0, v0, H, G, D, V, qn, kn, eps, inv_freq, rot, positions,
                                                                        slot_map, page, qout, (AT*)kpool, (AT*)vpool)));
  return last();
}

bool delta_scan_wants_prepare(int N, int max_q) { return N <= 256 && max_q >= kDeltaWarpMinTokens; }
long long delta_scan_prepare_width(int G, int H, int N, int P) { return delta_pre_width(G, H, N, P); }

int sink_attention_warps(int H, int G) {
  const int rg = H / G;
  return rg < 8 ? rg : 8;
}

template <typename AT, int NPL, bool VEC>
static cudaError_t sink_attention_t(const SinkAttnArgs& a, int T, cudaStream_t s) {
  const int nw = sink_attention_warps(a.H, a.G), nb = (a.H / a.G + nw - 1) / nw;
  const size_t smem = ((size_t)nw * a.D + (size_t)kTile * (a.D + (VEC ? 4 : 1)) + (size_t)kTile * a.V) * sizeof(float);
  auto k = sink_attention_kernel<AT, NPL, VEC>;
  if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
  k<<<dim3(T, a.G * nb, a.nsplit), 32 * nw, smem, s>>>(a);
  if (a.nsplit > 1) sink_combine_kernel<AT, NPL><<<T * a.H, 32, 0, s>>>(a.part, a.sink, a.H, a.V, a.nsplit, a.out_mult, (AT*)a.out, a.ld_out);
  return last();
}

cudaError_t sink_attention_launch(const float* q, const void* kpool, const void* vpool, const float* sink, const int* block_tables, int max_blocks,
                                  const int* positions, const int* cu, int B, int H, int G, int D, int V, int page, int block, int window,
                                  float scale, float out_mult, void* out, long long ld_out, bool f32, int T, int nsplit, int chunk, float* part,
                                  cudaStream_t s) {
  if (G < 1 || H % G != 0 || V > 512 || (size_t)(8 * D + kTile * (D + 4) + kTile * V) * sizeof(float) > 220 * 1024) return cudaErrorInvalidValue;
  SinkAttnArgs a{q, kpool, vpool, sink, block_tables, max_blocks, positions, cu, B, H, G, D, V, page, block, window, scale, out_mult, out, ld_out,
                 nsplit, chunk, part};
  const int npl = (V + 31) / 32;
  if (V % 128 == 0 && D % (f32 ? 4 : 8) == 0) {            // 16-byte path: whole chunks of keys, four adjacent value columns per lane
#define SINK_VEC(N) AT_DISPATCH(f32, return (sink_attention_t<AT, N, true>(a, T, s)))
    if (npl <= 4) SINK_VEC(4);
    if (npl <= 8) SINK_VEC(8);
    SINK_VEC(16);
#undef SINK_VEC
  }
#define SINK_CASE(N) AT_DISPATCH(f32, return (sink_attention_t<AT, N, false>(a, T, s)))
  if (npl <= 1) SINK_CASE(1);
  if (npl <= 2) SINK_CASE(2);
  if (npl <= 4) SINK_CASE(4);
  if (npl <= 8) SINK_CASE(8);
  SINK_CASE(16);
#undef SINK_CASE
  return cudaErrorInvalidValue;
}

cudaError_t group_softmax_topk_launch(const float* z, long long ld_z, const float* corr, int E, int top, int ng, int keep, int* idx, float* w, int T,
                                      cudaStream_t s) {
  if (top > E || ng < 1 || E % ng != 0 || keep < 1 || keep > ng || (size_t)(2 * E + ng) * sizeof(float) > 48 * 1024) return cudaErrorInvalidValue;
  group_softmax_topk_kernel<<<T, 32, (2 * E + ng) * sizeof(float), s>>>(z, ld_z, corr, E, top, ng, keep, idx, w);
  return last();
}
}  // namespace b200
