// Kernels of sandwich-norm stacks with differential attention: layer norms (weight and bias) on the fp32 residual stream — alone and
// fused with the scaled residual add between an output-side and an input-side norm —, the append of a step's keys and values to
// separate paged pools, and differential attention itself: two softmax maps per head over the same values, subtracted with one weight,
// then a per-head unit-RMS norm.
//
// Conventions as in hybrid.cu: a step is a ragged batch (rows cu_seqlens[b] .. cu_seqlens[b+1] belong to sequence b); activations are
// AT = bf16 (serving) or float (exact mode); the residual stream, norms, scores, softmax and the map difference are fp32 in both.
#include "diffattn.h"
#include "hybrid_common.cuh"

namespace b200 {
namespace {

// ---------------------------------------------------------------------------------------------------------- layer norms
// mean and 1 / sqrt(biased variance + eps) of row[0..n) (two passes over the row: no cancellation)
__device__ __forceinline__ void row_stats(const float* row, int n, float eps, float* red, float& mu, float& rstd) {
  float s = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) s += row[c];
  mu = block_sum(s, red) / (float)n;
  float v = 0.f;
  for (int c = threadIdx.x; c < n; c += blockDim.x) { const float d = row[c] - mu; v += d * d; }
  rstd = 1.f / sqrtf(block_sum(v, red) / (float)n + eps);
}

template <typename AT>
__global__ void layernorm_cast_kernel(const float* __restrict__ x, long long ld_x, const float* __restrict__ w, const float* __restrict__ b,
                                      AT* __restrict__ out, int n, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const float* row = x + t * ld_x;
  float mu, rstd;
  row_stats(row, n, eps, red, mu, rstd);
  for (int c = threadIdx.x; c < n; c += blockDim.x) stf<AT>(out + t * n + c, (row[c] - mu) * rstd * w[c] + b[c]);
}

// x += mult * LN(y; pw, pb)   (x, y fp32);   xa = (AT) LN(x; nw, nb)
template <typename AT>
__global__ void post_layernorm_add_norm_kernel(float* __restrict__ x, const float* __restrict__ y, long long ld_y, const float* __restrict__ pw,
                                               const float* __restrict__ pb, float mult, const float* __restrict__ nw,
                                               const float* __restrict__ nb, AT* __restrict__ xa, int n, float eps) {
  __shared__ float red[32];
  const long long t = blockIdx.x;
  const float* yr = y + t * ld_y;
  float* xr = x + t * n;
  float mu, rstd;
  row_stats(yr, n, eps, red, mu, rstd);
  for (int c = threadIdx.x; c < n; c += blockDim.x) xr[c] += mult * ((yr[c] - mu) * rstd * pw[c] + pb[c]);    // own writes: same thread, same c
  row_stats(xr, n, eps, red, mu, rstd);
  for (int c = threadIdx.x; c < n; c += blockDim.x) stf<AT>(xa + t * n + c, (xr[c] - mu) * rstd * nw[c] + nb[c]);
}

// ---------------------------------------------------------------------------------------------------------- key / value append
// row t of `rows` holds the keys of all G heads from column k0 on (G * dk wide) and the values from column v0 on (G * dv wide);
// they go to slot slot_map[t] = page * page_size + offset of the pools [pages, G, page_size, d]
template <typename AT>
__global__ void paged_kv_append_kernel(const AT* __restrict__ rows, long long ld, int k0, int v0, AT* __restrict__ kpool, AT* __restrict__ vpool,
                                       const int* __restrict__ slot_map, int G, int dk, int dv, int page) {
  const long long t = blockIdx.x;
  const int slot = slot_map[t], pg = slot / page, off = slot % page;
  const AT* r = rows + t * ld;
  for (int i = threadIdx.x; i < G * dk; i += blockDim.x) kpool[(((long long)pg * G + i / dk) * page + off) * dk + i % dk] = r[k0 + i];
  for (int i = threadIdx.x; i < G * dv; i += blockDim.x) vpool[(((long long)pg * G + i / dv) * page + off) * dv + i % dv] = r[v0 + i];
}

// ---------------------------------------------------------------------------------------------------------- differential attention
struct DiffAttnArgs {
  const void* q; long long ld_q;            // row t: head h, map c at q + t * ld_q + (h * 2 + c) * D
  const void* kpool; const void* vpool;     // [pages, G, page, 2D] (maps side by side) / [pages, G, page, V]
  const int* block_tables; int max_blocks;
  const int* positions; const int* cu; int B;
  int H, G, D, V, page;
  float scale, softcap, temp_coef, temp_every, lam, eps, out_mult;
  void* out;                                // AT [T, H * V]
  int nsplit, chunk;
  float* part;                              // [T, H, nsplit, 2, V + 2] = (m, l, o[V]) per map when the keys are split
};

constexpr int kDiffTile = 32;               // keys per tile: one per lane

// value column of register i of a lane: VEC (vdim a multiple of 128) 4 lane + 128 (i / 4) + i % 4 — four adjacent columns per 16-byte
// shared-memory load —, else lane + 32 i
template <bool VEC>
__device__ __forceinline__ int vcol(int lane, int i) { return VEC ? 4 * lane + 128 * (i >> 2) + (i & 3) : lane + 32 * i; }

// o = a1 - lam a2,  o / sqrt(mean(o^2) + eps) * out_mult
template <typename AT, int NPL, bool VEC>
__device__ __forceinline__ void diff_finish(const float* a1, const float* a2, int V, float lam, float eps, float out_mult, AT* orow, int lane) {
  float o[NPL], ss = 0.f;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int d = vcol<VEC>(lane, i);
    o[i] = d < V ? a1[i] - lam * a2[i] : 0.f;
    ss += o[i] * o[i];
  }
  const float r = out_mult / sqrtf(warp_sum(ss) / (float)V + eps);
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int d = vcol<VEC>(lane, i);
    if (d < V) stf<AT>(orow + d, o[i] * r);
  }
}

// grid (tokens, G * ceil((H/G) / warps), key splits); one warp per query head, the warps of a CTA share one key / value head whose
// tile of kDiffTile keys and values is staged in shared memory as floats.  Lane j scores key j of the tile for both maps; the two
// running softmaxes (m, l) and accumulators live in registers, each lane owning the value columns vcol(lane, i).
// VEC (2 dim a multiple of 8, vdim a multiple of 128): 16-byte shared-memory loads in both phases, key rows padded by 4 floats; else
// scalar loads, key rows padded by 1.
template <typename AT, int NPL, bool VEC>
__global__ void diff_attention_kernel(DiffAttnArgs a) {
  extern __shared__ __align__(16) float smem[];
  const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int D2 = 2 * a.D, V = a.V, ldk = VEC ? D2 + 4 : D2 + 1;
  float* qs = smem;                         // [nw][2D]
  float* ks = qs + nw * D2;                 // [tile][2D + 1]
  float* vs = ks + kDiffTile * ldk;         // [tile][V]
  const int t = blockIdx.x, Rg = a.H / a.G, nb = (Rg + nw - 1) / nw;
  const int g = blockIdx.y / nb, r = (blockIdx.y % nb) * nw + warp, h = g * Rg + r;
  const bool valid = r < Rg;
  const int pos = a.positions[t];
  const int* bt = a.block_tables + (long long)seq_of(a.cu, a.B, t) * a.max_blocks;
  const AT* qrow = (const AT*)a.q + (long long)t * a.ld_q;
  for (int i = threadIdx.x; i < nw * D2; i += blockDim.x) {
    const int rr = (blockIdx.y % nb) * nw + i / D2;
    qs[i] = rr < Rg ? ldf<AT>(qrow + (long long)(g * Rg + rr) * D2 + i % D2) : 0.f;
  }
  const float mul = a.temp_coef != 0.f ? a.scale * (1.f + a.temp_coef * logf(floorf((float)(pos + 1) / a.temp_every) + 1.f)) : a.scale;
  float m1 = -INFINITY, m2 = -INFINITY, l1 = 0.f, l2 = 0.f, o1[NPL], o2[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) o1[i] = o2[i] = 0.f;
  const float* qh = qs + warp * D2;
  const int jbeg = blockIdx.z * a.chunk, jend = (int)min((long long)pos + 1, (long long)jbeg + a.chunk);
  constexpr int E = 16 / (int)sizeof(AT);
  const bool vec = D2 % E == 0 && V % E == 0;
  // VEC: each thread keeps up to kPrefetch 16-byte chunks of the NEXT tile in registers while the current one is scored; what does not
  // fit is fetched when the tile is staged.  Chunk id = row * cpr + column (keys first, then values).  The block-table entries of this
  // CTA's key range sit in shared memory, so a chunk's address does not wait for another global load.
  constexpr int kPrefetch = VEC ? 8 : 1;
  uint4 pre[kPrefetch];
  const int cpr = (D2 + V) / E, kc = D2 / E, nthr = blockDim.x;
  const unsigned cpr_inv = (unsigned)((0x100000000ull + cpr - 1) / cpr);          // id / cpr == umulhi(id, cpr_inv) for id < 2^16
  int* bts = reinterpret_cast<int*>(vs + kDiffTile * V);
  const int pg0 = jbeg / a.page;
  const bool tile_in_page = a.page % kDiffTile == 0;                               // jbeg is a multiple of the tile
  auto tile_row0 = [&](int j0) -> long long { return ((long long)bts[j0 / a.page - pg0] * a.G + g) * a.page + j0 % a.page; };
  auto chunk_src = [&](long long row0, int j0, int jj, int cc) -> const uint4* {
    const long long row = tile_in_page ? row0 + jj : tile_row0(j0 + jj);
    return reinterpret_cast<const uint4*>(cc < kc ? (const AT*)a.kpool + row * D2 + cc * E : (const AT*)a.vpool + row * V + (cc - kc) * E);
  };
  auto chunk_put = [&](int jj, int cc, const uint4& v) {
    float f[E];
    unpack16<AT>(v, f);
    float* dst = cc < kc ? ks + jj * ldk + cc * E : vs + jj * V + (cc - kc) * E;
#pragma unroll
    for (int e = 0; e < E; e += 4) *reinterpret_cast<float4*>(dst + e) = make_float4(f[e], f[e + 1], f[e + 2], f[e + 3]);
  };
  auto prefetch = [&](int j0, int nk) {
    const long long row0 = tile_in_page ? tile_row0(j0) : 0;
#pragma unroll
    for (int u = 0; u < kPrefetch; ++u) {
      const int id = threadIdx.x + u * nthr;
      if (id < nk * cpr) { const int jj = __umulhi((unsigned)id, cpr_inv); pre[u] = *chunk_src(row0, j0, jj, id - jj * cpr); }
    }
  };
  if (VEC) {
    if (jbeg < jend)
      for (int i = threadIdx.x; i <= (jend - 1) / a.page - pg0; i += nthr) bts[i] = bt[pg0 + i];
    __syncthreads();
    if (jbeg < jend) prefetch(jbeg, min(kDiffTile, jend - jbeg));
  }
  for (int j0 = jbeg; j0 < jend; j0 += kDiffTile) {
    __syncthreads();
    const int nk = min(kDiffTile, jend - j0);
    if (VEC) {
#pragma unroll
      for (int u = 0; u < kPrefetch; ++u) {
        const int id = threadIdx.x + u * nthr;
        if (id < nk * cpr) { const int jj = __umulhi((unsigned)id, cpr_inv); chunk_put(jj, id - jj * cpr, pre[u]); }
      }
      if (kPrefetch * nthr < nk * cpr) {
        const long long row0 = tile_in_page ? tile_row0(j0) : 0;
        for (int id = kPrefetch * nthr + threadIdx.x; id < nk * cpr; id += nthr) {
          const int jj = __umulhi((unsigned)id, cpr_inv), cc = id - jj * cpr;
          chunk_put(jj, cc, *chunk_src(row0, j0, jj, cc));
        }
      }
    } else {
      for (int jj = warp; jj < nk; jj += nw) {          // each warp fetches whole rows: one block-table lookup per row
        const int j = j0 + jj;
        const long long base = ((long long)bt[j / a.page] * a.G + g) * a.page + j % a.page;
        const AT* ksrc = (const AT*)a.kpool + base * D2;
        const AT* vsrc = (const AT*)a.vpool + base * V;
        float* kd = ks + jj * ldk;
        float* vd = vs + jj * V;
        if (vec) {
          for (int c = lane; c < D2 / E; c += 32) unpack16<AT>(*reinterpret_cast<const uint4*>(ksrc + c * E), kd + c * E);
          for (int c = lane; c < V / E; c += 32) unpack16<AT>(*reinterpret_cast<const uint4*>(vsrc + c * E), vd + c * E);
        } else {
          for (int d = lane; d < D2; d += 32) kd[d] = ldf<AT>(ksrc + d);
          for (int d = lane; d < V; d += 32) vd[d] = ldf<AT>(vsrc + d);
        }
      }
    }
    __syncthreads();
    if (VEC && j0 + kDiffTile < jend) prefetch(j0 + kDiffTile, min(kDiffTile, jend - j0 - kDiffTile));
    if (!valid) continue;
    float s1 = -INFINITY, s2 = -INFINITY;
    if (lane < nk) {
      const float* kr = ks + lane * ldk;
      float d1 = 0.f, d2 = 0.f;
      if (VEC) {
        const float4* q4 = reinterpret_cast<const float4*>(qh);
        const float4* k4 = reinterpret_cast<const float4*>(kr);
        const int n4 = a.D >> 2;
        for (int d = 0; d < n4; ++d) {
          const float4 x = q4[d], y = k4[d], z = q4[n4 + d], w = k4[n4 + d];
          d1 += x.x * y.x + x.y * y.y + x.z * y.z + x.w * y.w;
          d2 += z.x * w.x + z.y * w.y + z.z * w.z + z.w * w.w;
        }
      } else {
        for (int d = 0; d < a.D; ++d) { d1 += qh[d] * kr[d]; d2 += qh[a.D + d] * kr[a.D + d]; }
      }
      s1 = d1 * mul; s2 = d2 * mul;
      if (a.softcap > 0.f) { s1 = a.softcap * tanhf(s1 / a.softcap); s2 = a.softcap * tanhf(s2 / a.softcap); }
    }
    const float n1 = fmaxf(m1, warp_max(s1)), n2 = fmaxf(m2, warp_max(s2));
    const float c1 = m1 == -INFINITY ? 0.f : expf(m1 - n1), c2 = m2 == -INFINITY ? 0.f : expf(m2 - n2);
    const float p1 = lane < nk ? expf(s1 - n1) : 0.f, p2 = lane < nk ? expf(s2 - n2) : 0.f;
    l1 = l1 * c1 + warp_sum(p1); l2 = l2 * c2 + warp_sum(p2);
    m1 = n1; m2 = n2;
#pragma unroll
    for (int i = 0; i < NPL; ++i) { o1[i] *= c1; o2[i] *= c2; }
    for (int jj = 0; jj < nk; ++jj) {
      const float w1 = __shfl_sync(0xffffffffu, p1, jj), w2 = __shfl_sync(0xffffffffu, p2, jj);
      const float* vr = vs + jj * V;
      if (VEC) {
#pragma unroll
        for (int i = 0; i < NPL / 4; ++i)
          if (128 * i < V) {
            const float4 c = *reinterpret_cast<const float4*>(vr + 4 * lane + 128 * i);
            o1[4 * i] += w1 * c.x; o1[4 * i + 1] += w1 * c.y; o1[4 * i + 2] += w1 * c.z; o1[4 * i + 3] += w1 * c.w;
            o2[4 * i] += w2 * c.x; o2[4 * i + 1] += w2 * c.y; o2[4 * i + 2] += w2 * c.z; o2[4 * i + 3] += w2 * c.w;
          }
      } else {
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          const int d = lane + 32 * i;
          if (d < V) { const float v = vr[d]; o1[i] += w1 * v; o2[i] += w2 * v; }
        }
      }
    }
  }
  if (!valid) return;
  if (a.nsplit == 1) {
    const float i1 = 1.f / l1, i2 = 1.f / l2;          // the query's own position is always visible: l > 0
#pragma unroll
    for (int i = 0; i < NPL; ++i) { o1[i] *= i1; o2[i] *= i2; }
    diff_finish<AT, NPL, VEC>(o1, o2, V, a.lam, a.eps, a.out_mult, (AT*)a.out + ((long long)t * a.H + h) * V, lane);
  } else {
    float* pp = a.part + (((long long)t * a.H + h) * a.nsplit + blockIdx.z) * 2 * (V + 2);
    if (lane == 0) { pp[0] = m1; pp[1] = l1; pp[V + 2] = m2; pp[V + 3] = l2; }
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = vcol<VEC>(lane, i);
      if (d < V) { pp[2 + d] = o1[i]; pp[V + 4 + d] = o2[i]; }
    }
  }
}

// merge the key splits of one (token, head), map by map: a = sum_z o_z e^(m_z - M) / sum_z l_z e^(m_z - M); then the difference and
// its norm.  One warp per (token, head).
template <typename AT, int NPL>
__global__ void diff_combine_kernel(const float* __restrict__ part, int V, int nsplit, float lam, float eps, float out_mult, AT* __restrict__ out) {
  const long long th = blockIdx.x;
  const int lane = threadIdx.x;
  float acc[2][NPL];
  for (int c = 0; c < 2; ++c) {
    const float* pp = part + th * nsplit * 2 * (V + 2) + c * (V + 2);
    float M = -INFINITY, den = 0.f;
    for (int z = 0; z < nsplit; ++z) M = fmaxf(M, pp[(long long)z * 2 * (V + 2)]);
#pragma unroll
    for (int i = 0; i < NPL; ++i) acc[c][i] = 0.f;
    for (int z = 0; z < nsplit; ++z) {
      const float* pz = pp + (long long)z * 2 * (V + 2);
      if (pz[0] == -INFINITY) continue;               // a split beyond this token's keys
      const float e = expf(pz[0] - M);
      den += pz[1] * e;
#pragma unroll
      for (int i = 0; i < NPL; ++i) { const int d = lane + 32 * i; if (d < V) acc[c][i] += pz[2 + d] * e; }
    }
    const float inv = 1.f / den;
#pragma unroll
    for (int i = 0; i < NPL; ++i) acc[c][i] *= inv;
  }
  diff_finish<AT, NPL, false>(acc[0], acc[1], V, lam, eps, out_mult, out + th * V, lane);
}

// prefill as matrix products: a1, a2 fp32 [G, 2, T * Rg, V] (row t * Rg + r of block (g, c) = token t, head g * Rg + r, map c) ->
// out[t, (g * Rg + r) * V + d].  One warp per (token, head).
template <typename AT, int NPL>
__global__ void diff_head_norm_kernel(const float* __restrict__ a, int T, int H, int G, int V, float lam, float eps, float out_mult,
                                      AT* __restrict__ out) {
  const long long th = blockIdx.x;
  const int t = (int)(th / H), h = (int)(th % H), Rg = H / G, g = h / Rg, r = h % Rg, lane = threadIdx.x;
  const float* p1 = a + (((long long)g * 2) * T * Rg + (long long)t * Rg + r) * V;
  const float* p2 = p1 + (long long)T * Rg * V;
  float a1[NPL], a2[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) { const int d = lane + 32 * i; a1[i] = d < V ? p1[d] : 0.f; a2[i] = d < V ? p2[d] : 0.f; }
  diff_finish<AT, NPL, false>(a1, a2, V, lam, eps, out_mult, out + th * V, lane);
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------- launchers
cudaError_t layernorm_cast_launch(const float* x, long long ld_x, const float* w, const float* b, void* out, bool f32, int n, float eps, int T,
                                  cudaStream_t s) {
  AT_DISPATCH(f32, (layernorm_cast_kernel<AT><<<T, 256, 0, s>>>(x, ld_x, w, b, (AT*)out, n, eps)));
  return last();
}

cudaError_t post_layernorm_add_norm_launch(float* x, const float* y, long long ld_y, const float* pw, const float* pb, float mult, const float* nw,
                                           const float* nb, void* xa, bool f32, int n, float eps, int T, cudaStream_t s) {
  AT_DISPATCH(f32, (post_layernorm_add_norm_kernel<AT><<<T, 256, 0, s>>>(x, y, ld_y, pw, pb, mult, nw, nb, (AT*)xa, n, eps)));
  return last();
}

cudaError_t paged_kv_append_launch(const void* rows, long long ld, int k0, int v0, void* kpool, void* vpool, const int* slot_map, int G, int dk,
                                   int dv, int page, bool f32, int T, cudaStream_t s) {
  AT_DISPATCH(f32, (paged_kv_append_kernel<AT><<<T, 256, 0, s>>>((const AT*)rows, ld, k0, v0, (AT*)kpool, (AT*)vpool, slot_map, G, dk, dv, page)));
  return last();
}

int diff_attention_warps(int H, int G) {
  const int Rg = H / G;
  return Rg < 1 ? 1 : (Rg > 8 ? 8 : Rg);
}

template <typename AT, int NPL, bool VEC>
static cudaError_t diff_attention_launch_v(const DiffAttnArgs& a, int T, cudaStream_t s) {
  const int nw = diff_attention_warps(a.H, a.G), Rg = a.H / a.G, nb = (Rg + nw - 1) / nw;
  // VEC also keeps the block-table entries of the CTA's key range: all of the table with one split, chunk / page + 2 with more
  const size_t nbt = VEC ? (size_t)(a.nsplit == 1 ? a.max_blocks : (a.chunk / a.page + 2 < a.max_blocks ? a.chunk / a.page + 2 : a.max_blocks)) : 0;
  const size_t smem = ((size_t)nw * 2 * a.D + (size_t)kDiffTile * (2 * a.D + (VEC ? 4 : 1)) + (size_t)kDiffTile * a.V + nbt) * sizeof(float);
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  auto k = diff_attention_kernel<AT, NPL, VEC>;
  if (smem > 48 * 1024) { cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); if (e != cudaSuccess) return e; }
  k<<<dim3(T, a.G * nb, a.nsplit), nw * 32, smem, s>>>(a);
  cudaError_t e = last();
  if (e != cudaSuccess || a.nsplit == 1) return e;
  diff_combine_kernel<AT, NPL><<<T * a.H, 32, 0, s>>>(a.part, a.V, a.nsplit, a.lam, a.eps, a.out_mult, (AT*)a.out);
  return last();
}

template <typename AT, int NPL>
static cudaError_t diff_attention_launch_t(const DiffAttnArgs& a, int T, cudaStream_t s) {
  if (NPL % 4 == 0 && (2 * a.D) % 8 == 0 && a.V % 128 == 0) return diff_attention_launch_v<AT, NPL, true>(a, T, s);
  return diff_attention_launch_v<AT, NPL, false>(a, T, s);
}

cudaError_t diff_attention_launch(const void* q, long long ld_q, const void* kpool, const void* vpool, const int* block_tables, int max_blocks,
                                  const int* positions, const int* cu, int B, int H, int G, int D, int V, int page, float scale, float softcap,
                                  float temp_coef, float temp_every, float lam, float eps, float out_mult, void* out, bool f32, int T, int nsplit,
                                  int chunk, float* part, cudaStream_t s) {
  if (G < 1 || H % G != 0 || V < 1 || V > 512 || D < 1) return cudaErrorInvalidValue;
  DiffAttnArgs a{q, ld_q, kpool, vpool, block_tables, max_blocks, positions, cu, B, H, G, D, V, page, scale, softcap, temp_coef, temp_every,
                 lam, eps, out_mult, out, nsplit, chunk, part};
  if (V <= 128) { AT_DISPATCH(f32, return (diff_attention_launch_t<AT, 4>(a, T, s))); }
  if (V <= 256) { AT_DISPATCH(f32, return (diff_attention_launch_t<AT, 8>(a, T, s))); }
  AT_DISPATCH(f32, return (diff_attention_launch_t<AT, 16>(a, T, s)));
  return cudaErrorInvalidValue;
}

cudaError_t diff_head_norm_launch(const float* a, int T, int H, int G, int V, float lam, float eps, float out_mult, void* out, bool f32,
                                  cudaStream_t s) {
  if (V > 512 || H % G != 0) return cudaErrorInvalidValue;
  if (V <= 128) AT_DISPATCH(f32, (diff_head_norm_kernel<AT, 4><<<T * H, 32, 0, s>>>(a, T, H, G, V, lam, eps, out_mult, (AT*)out)));
  else if (V <= 256) AT_DISPATCH(f32, (diff_head_norm_kernel<AT, 8><<<T * H, 32, 0, s>>>(a, T, H, G, V, lam, eps, out_mult, (AT*)out)));
  else AT_DISPATCH(f32, (diff_head_norm_kernel<AT, 16><<<T * H, 32, 0, s>>>(a, T, H, G, V, lam, eps, out_mult, (AT*)out)));
  return last();
}

}  // namespace b200
