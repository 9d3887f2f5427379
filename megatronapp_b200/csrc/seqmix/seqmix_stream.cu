// Kernels of layers over several fp32 residual streams with a sliding-window attention beside a selective scan (sm_100a):
// the stream update fused with the layer norm of the next sublayer's input, sinusoidal positions added to an fp32 embedding, an
// RMS norm per head, paged grouped-query attention with a distance penalty per head, a sliding window, an optional sink in the
// softmax denominator and a scalar output gate per head, and the selective scan (one decay per channel and state).
//
// Conventions as in seqmix.cu: activations are `T` (float or __nv_bfloat16); statistics, angles, scores, weights, gates, decays,
// step sizes and every recurrent state are fp32; `cu[R + 1]` / `rows[R]` describe the packed batch.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <algorithm>

#include "seq_common.cuh"
#include "seqmix_api.h"

namespace b200seq {

namespace {

using namespace dev;

#define SEQ_DISPATCH_T(is_bf16, ...)                      \
  if (is_bf16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else { using T = float; __VA_ARGS__; }

__device__ __forceinline__ float block_sum(float v, float* red) {   // every thread gets the sum; red holds >= 32 floats
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
  return tot;
}

// ---------------------------------------------------------------------------------------------------------------------
// Streams X [T, S, W] (fp32, in place).  With a pending sublayer output: y = ls * (sa * (a + bias_a) + sb * b) and
// X_t <- sum_s mix[s, t] X_s + out[t] * y for all t at once.  Then, with `inp`: u = sum_s inp[s] X_s and
// h = (u - mean) / sqrt(var + eps) * w + beta (or u / sqrt(mean(u^2) + eps) * w without beta).  One CTA per token.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kMaxStreams = 16;

template <typename T>
__global__ void __launch_bounds__(256) stream_mix_norm_kernel(StreamNormArgs p) {
  extern __shared__ float su[];                      // [W]
  __shared__ float red[32];
  __shared__ float cmix[kMaxStreams * kMaxStreams], cout_[kMaxStreams], cin[kMaxStreams];
  const int S = p.S, W = p.W;
  if (threadIdx.x < S * S && p.mix != nullptr) cmix[threadIdx.x] = p.mix[threadIdx.x];
  if (threadIdx.x < S) {
    if (p.outc != nullptr) cout_[threadIdx.x] = p.outc[threadIdx.x];
    if (p.inp != nullptr) cin[threadIdx.x] = p.inp[threadIdx.x];
  }
  __syncthreads();
  const int64_t row = blockIdx.x;
  float* X = p.x + row * S * W;
  const T* a = static_cast<const T*>(p.a);
  const T* b = static_cast<const T*>(p.b);
  const T* ba = static_cast<const T*>(p.bias_a);
  const T* ls = static_cast<const T*>(p.ls);
  float sum = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float xs[kMaxStreams];
#pragma unroll
    for (int s = 0; s < kMaxStreams; ++s) xs[s] = s < S ? X[static_cast<int64_t>(s) * W + c] : 0.f;
    if (a != nullptr) {
      float y = ld(a + row * p.lda + c);
      if (ba != nullptr) y += ld(ba + c);
      y *= p.scale_a;
      if (b != nullptr) y = fmaf(p.scale_b, ld(b + row * p.ldb + c), y);
      if (ls != nullptr) y *= ld(ls + c);
      float nx[kMaxStreams];
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t) {
        if (t < S) {
          float v = cout_[t] * y;
#pragma unroll
          for (int s = 0; s < kMaxStreams; ++s)
            if (s < S) v = fmaf(cmix[s * S + t], xs[s], v);
          nx[t] = v;
        }
      }
#pragma unroll
      for (int t = 0; t < kMaxStreams; ++t)
        if (t < S) { xs[t] = nx[t]; X[static_cast<int64_t>(t) * W + c] = nx[t]; }
    }
    if (p.inp != nullptr) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < kMaxStreams; ++s)
        if (s < S) u = fmaf(cin[s], xs[s], u);
      su[c] = u;
      sum += u;
    }
  }
  if (p.inp == nullptr) return;
  const T* w = static_cast<const T*>(p.w);
  const T* beta = static_cast<const T*>(p.beta);
  T* h = static_cast<T*>(p.h) + row * W;
  float mean = 0.f;
  if (beta != nullptr || p.center) mean = block_sum(sum, red) / static_cast<float>(W);
  else __syncthreads();
  float ss = 0.f;
  for (int c = threadIdx.x; c < W; c += blockDim.x) { const float d = su[c] - mean; ss = fmaf(d, d, ss); }
  const float rstd = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(W) + p.eps);
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float v = (su[c] - mean) * rstd * ld(w + c);
    if (beta != nullptr) v += ld(beta + c);
    st(h + c, v);
  }
}

// Four columns per thread and the number of streams known at compile time (W a multiple of 4, rows 16-byte aligned).
template <typename T> __device__ __forceinline__ float4 ld4(const T* p);
template <> __device__ __forceinline__ float4 ld4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 ld4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void st4(T* p, float4 v);
template <> __device__ __forceinline__ void st4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void st4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  uint2 raw;
  *reinterpret_cast<__nv_bfloat162*>(&raw.x) = __floats2bfloat162_rn(v.x, v.y);
  *reinterpret_cast<__nv_bfloat162*>(&raw.y) = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float4 f4_fma(float a, float4 x, float4 y) {
  return make_float4(fmaf(a, x.x, y.x), fmaf(a, x.y, y.y), fmaf(a, x.z, y.z), fmaf(a, x.w, y.w));
}
__device__ __forceinline__ float4 f4_mul(float4 x, float4 y) { return make_float4(x.x * y.x, x.y * y.y, x.z * y.z, x.w * y.w); }

template <typename T, int S>
__global__ void __launch_bounds__(256) stream_mix_norm_vec_kernel(StreamNormArgs p) {
  extern __shared__ __align__(16) float su[];        // [W]
  __shared__ float red[32];
  const int W = p.W;
  const int64_t row = blockIdx.x;
  float* X = p.x + row * S * W;
  const T* a = static_cast<const T*>(p.a);
  const T* b = static_cast<const T*>(p.b);
  const T* ba = static_cast<const T*>(p.bias_a);
  const T* ls = static_cast<const T*>(p.ls);
  float cmix[S * S], cout_[S], cin[S];
#pragma unroll
  for (int i = 0; i < S * S; ++i) cmix[i] = a != nullptr ? p.mix[i] : 0.f;
#pragma unroll
  for (int i = 0; i < S; ++i) { cout_[i] = a != nullptr ? p.outc[i] : 0.f; cin[i] = p.inp != nullptr ? p.inp[i] : 0.f; }
  float sum = 0.f;
  for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
    float4 xs[S];
#pragma unroll
    for (int s = 0; s < S; ++s) xs[s] = *reinterpret_cast<const float4*>(X + static_cast<int64_t>(s) * W + c);
    if (a != nullptr) {
      float4 y = ld4(a + row * p.lda + c);
      if (ba != nullptr) { const float4 bv = ld4(ba + c); y = make_float4(y.x + bv.x, y.y + bv.y, y.z + bv.z, y.w + bv.w); }
      y = make_float4(y.x * p.scale_a, y.y * p.scale_a, y.z * p.scale_a, y.w * p.scale_a);
      if (b != nullptr) y = f4_fma(p.scale_b, ld4(b + row * p.ldb + c), y);
      if (ls != nullptr) y = f4_mul(y, ld4(ls + c));
      float4 nx[S];
#pragma unroll
      for (int t = 0; t < S; ++t) {
        float4 v = make_float4(cout_[t] * y.x, cout_[t] * y.y, cout_[t] * y.z, cout_[t] * y.w);
#pragma unroll
        for (int s = 0; s < S; ++s) v = f4_fma(cmix[s * S + t], xs[s], v);
        nx[t] = v;
      }
#pragma unroll
      for (int t = 0; t < S; ++t) { xs[t] = nx[t]; *reinterpret_cast<float4*>(X + static_cast<int64_t>(t) * W + c) = nx[t]; }
    }
    if (p.inp != nullptr) {
      float4 u = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int s = 0; s < S; ++s) u = f4_fma(cin[s], xs[s], u);
      *reinterpret_cast<float4*>(su + c) = u;
      sum += (u.x + u.y) + (u.z + u.w);
    }
  }
  if (p.inp == nullptr) return;
  const T* w = static_cast<const T*>(p.w);
  const T* beta = static_cast<const T*>(p.beta);
  T* h = static_cast<T*>(p.h) + row * W;
  float mean = 0.f;
  if (beta != nullptr || p.center) mean = block_sum(sum, red) / static_cast<float>(W);
  else __syncthreads();
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
    const float4 u = *reinterpret_cast<const float4*>(su + c);
    const float d0 = u.x - mean, d1 = u.y - mean, d2 = u.z - mean, d3 = u.w - mean;
    ss += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
  }
  const float rstd = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(W) + p.eps);
  for (int c = threadIdx.x * 4; c < W; c += blockDim.x * 4) {
    const float4 u = *reinterpret_cast<const float4*>(su + c);
    const float4 wv = ld4(w + c);
    float4 v = make_float4((u.x - mean) * rstd * wv.x, (u.y - mean) * rstd * wv.y, (u.z - mean) * rstd * wv.z, (u.w - mean) * rstd * wv.w);
    if (beta != nullptr) { const float4 bv = ld4(beta + c); v = make_float4(v.x + bv.x, v.y + bv.y, v.z + bv.z, v.w + bv.w); }
    st4(h + c, v);
  }
}

// x [T, W] (fp32, in place): x[t, 2i] += sin(pos_t * f_i), x[t, 2i + 1] += cos(pos_t * f_i)
__global__ void add_sinusoid_kernel(float* __restrict__ x, const int64_t* __restrict__ positions, const float* __restrict__ freq,
                                    int64_t n_pairs_total, int half) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n_pairs_total) return;
  const int64_t t = idx / half;
  const int i = static_cast<int>(idx % half);
  const float ang = static_cast<float>(positions[t]) * freq[i];
  float sn, cs;
  sincosf(ang, &sn, &cs);
  float2* px = reinterpret_cast<float2*>(x + t * (2 * static_cast<int64_t>(half))) + i;
  float2 v = *px;
  v.x += sn; v.y += cs;
  *px = v;
}

// x [T, heads, d] (row stride ldx) -> y contiguous: every head divided by its root mean square over d, times w [d]
template <typename T>
__global__ void __launch_bounds__(128) head_rms_norm_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w,
                                                            T* __restrict__ y, int64_t rows, int heads, int d, float eps) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int64_t t = row / heads;
  const int h = static_cast<int>(row % heads);
  const T* src = x + t * ldx + static_cast<int64_t>(h) * d;
  float ss = 0.f;
  for (int c = lane; c < d; c += 32) { const float v = ld(src + c); ss = fmaf(v, v, ss); }
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(d) + eps);
  for (int c = lane; c < d; c += 32) st(y + row * d + c, ld(src + c) * r * ld(w + c));
}

// ---------------------------------------------------------------------------------------------------------------------
// Paged grouped-query attention with a sliding window.  Query at position i sees keys j with 0 <= i - j < window (window 0:
// all keys up to i); score = q . k * scale - slope[h] * (i - j) + dist_bias[min(i - j, n_bias - 1)][h]; weights exp(s_j) / (sink + sum_j exp(s_j)) where the sink
// (0 or 1) is a key of score 0 without a value; the head's output is multiplied by sigmoid(gate[t, h]) and out_scale.
//
// grid (query blocks, kv heads, head chunks x key splits).  A CTA takes QB consecutive packed tokens and HC heads of one kv
// head: its QB * HC <= 64 (query, head) pairs are dealt round robin to 8 warps, up to 8 per warp.  Keys and values of a tile of
// 32 cached tokens are staged in shared memory as fp32 once for all pairs.  Scores: a lane owns one key of the tile and walks
// the head dimension for all pairs of its warp at once (the queries of a warp lie pair-interleaved, so one 16-byte broadcast
// read brings a channel of four pairs); the online softmax state (m, l) is kept per pair; values: a lane owns channels
// lane, lane + 32, ... of the accumulators.  A block of tokens that straddles sequences walks them one after the other.
// Decoding batches (one token per sequence) run window_attention_decode_kernel below.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kWinWarps = 8, kWinSlots = 8, kWinTile = 32;

template <typename T>
__device__ __forceinline__ void stage_rows(float* dst, int ld_dst, const T* cache, const int* table, int block_size, int G, int g,
                                           int width, int k0, int n_keys) {
  for (int i = threadIdx.x; i < n_keys * width; i += blockDim.x) {
    const int j = i / width, c = i % width, key = k0 + j;
    const int64_t slot = static_cast<int64_t>(table[key / block_size]) * block_size + key % block_size;
    dst[j * ld_dst + c] = ld(cache + (slot * G + g) * width + c);
  }
}
// 16-byte loads of bf16 rows (width a multiple of 8, rows 16-byte aligned)
__device__ __forceinline__ void stage_rows_vec(float* dst, int ld_dst, const __nv_bfloat16* cache, const int* table, int block_size,
                                               int G, int g, int width, int k0, int n_keys) {
  const int per_row = width >> 3;
  for (int i = threadIdx.x; i < n_keys * per_row; i += blockDim.x) {
    const int j = i / per_row, c = (i % per_row) << 3, key = k0 + j;
    const int64_t slot = static_cast<int64_t>(table[key / block_size]) * block_size + key % block_size;
    const uint4 raw = *reinterpret_cast<const uint4*>(cache + (slot * G + g) * width + c);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
    float* o = dst + j * ld_dst + c;
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h2[e]); o[2 * e] = f.x; o[2 * e + 1] = f.y; }
  }
}
template <typename T>
__device__ __forceinline__ void stage_tile(float* dst, int ld_dst, const T* cache, const int* table, int block_size, int G, int g,
                                           int width, int k0, int n_keys, bool vec) {
  stage_rows<T>(dst, ld_dst, cache, table, block_size, G, g, width, k0, n_keys);
}
template <>
__device__ __forceinline__ void stage_tile<__nv_bfloat16>(float* dst, int ld_dst, const __nv_bfloat16* cache, const int* table,
                                                          int block_size, int G, int g, int width, int k0, int n_keys, bool vec) {
  if (vec) stage_rows_vec(dst, ld_dst, cache, table, block_size, G, g, width, k0, n_keys);
  else stage_rows<__nv_bfloat16>(dst, ld_dst, cache, table, block_size, G, g, width, k0, n_keys);
}

template <typename T, int DVR>
__global__ void __launch_bounds__(kWinWarps * 32) window_attention_kernel(WindowAttnArgs p) {
  constexpr int NW = kWinWarps;
  extern __shared__ __align__(16) float smem[];
  const int d = p.d, dv = p.dv, ldk = d + 1, ldv = dv;
  float* sq = smem;                                        // [warps][d][slots]
  float* sk = sq + NW * kWinSlots * d;              // [tile][d + 1]
  float* sv = sk + kWinTile * ldk;                         // [tile][dv]
  float* sp = sv + kWinTile * ldv;                         // [warps][tile][slots]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.y, rep = p.H / p.G;
  const int h_lo = blockIdx.z * p.HC, n_heads = min(p.HC, rep - h_lo);     // heads of this chunk, relative to the group
  const int t0 = blockIdx.x * p.QB, t1 = min(p.n_tok, t0 + p.QB);
  const T* qbase = static_cast<const T*>(p.q);
  const T* kc = static_cast<const T*>(p.kcache);
  const T* vc = static_cast<const T*>(p.vcache);
  const bool vec_k = (d & 7) == 0, vec_v = (dv & 7) == 0;
  float* mysp = sp + warp * kWinTile * kWinSlots;
  const float* myq = sq + warp * kWinSlots * d;

  int seg = t0;
  while (seg < t1) {
    const int r = p.tok_req[seg];
    int seg_end = seg + 1;
    while (seg_end < t1 && p.tok_req[seg_end] == r) ++seg_end;
    const int nq = seg_end - seg, n_pairs = nq * n_heads;
    const int ns = warp < n_pairs ? (n_pairs - warp + NW - 1) / NW : 0;       // pairs of this warp
    const int* table = p.block_table + static_cast<int64_t>(r) * p.max_blocks;
    const int len_first = p.tok_len[seg], len_last = p.tok_len[seg_end - 1];
    const int k_begin = p.window > 0 ? max(0, len_first - p.window) : 0, k_end = len_last;
    __syncthreads();                                       // the previous segment's reads of sq are over
    for (int i = threadIdx.x; i < n_pairs * d; i += blockDim.x) {
      const int pr = i / d, c = i % d, qi = pr / n_heads, hh = pr % n_heads;
      sq[((pr % NW) * d + c) * kWinSlots + pr / NW] =
          ld(qbase + static_cast<int64_t>(seg + qi) * p.ldq + static_cast<int64_t>(g * rep + h_lo + hh) * d + c) * p.scale;
    }
    float m[kWinSlots], l[kWinSlots], acc[kWinSlots][DVR], slope[kWinSlots];
    int pos[kWinSlots], lo[kWinSlots], hd[kWinSlots];
    const bool with_sink = p.sink != 0;
#pragma unroll
    for (int u = 0; u < kWinSlots; ++u) {
      m[u] = with_sink ? 0.f : -INFINITY;
      l[u] = with_sink ? 1.f : 0.f;
#pragma unroll
      for (int k = 0; k < DVR; ++k) acc[u][k] = 0.f;
      pos[u] = -1; lo[u] = 0; slope[u] = 0.f; hd[u] = 0;
      if (u < ns) {
        const int pr = warp + u * NW, qi = pr / n_heads, hh = pr % n_heads;
        hd[u] = g * rep + h_lo + hh;
        pos[u] = p.tok_len[seg + qi] - 1;
        lo[u] = p.window > 0 ? max(0, pos[u] + 1 - p.window) : 0;
        slope[u] = p.slopes != nullptr ? p.slopes[g * rep + h_lo + hh] : 0.f;
      }
    }
    for (int k0 = k_begin; k0 < k_end; k0 += kWinTile) {
      const int n_keys = min(kWinTile, k_end - k0);
      __syncthreads();                                     // the previous tile (and sq) is settled
      stage_tile<T>(sk, ldk, kc, table, p.block_size, p.G, g, d, k0, n_keys, vec_k);
      stage_tile<T>(sv, ldv, vc, table, p.block_size, p.G, g, dv, k0, n_keys, vec_v);
      __syncthreads();
      bool any = false;                                    // does any pair of this warp see a key of this tile?
#pragma unroll
      for (int u = 0; u < kWinSlots; ++u) any = any || (u < ns && pos[u] >= k0 && lo[u] < k0 + n_keys);
      if (!any) continue;
      float s[kWinSlots];
#pragma unroll
      for (int u = 0; u < kWinSlots; ++u) s[u] = 0.f;
      if (lane < n_keys) {
        const float* krow = sk + lane * ldk;
        if (ns > 4) {
          for (int c = 0; c < d; ++c) {
            const float kv = krow[c];
            const float4 qa = *reinterpret_cast<const float4*>(myq + c * kWinSlots);
            const float4 qb = *reinterpret_cast<const float4*>(myq + c * kWinSlots + 4);
            s[0] = fmaf(qa.x, kv, s[0]); s[1] = fmaf(qa.y, kv, s[1]); s[2] = fmaf(qa.z, kv, s[2]); s[3] = fmaf(qa.w, kv, s[3]);
            s[4] = fmaf(qb.x, kv, s[4]); s[5] = fmaf(qb.y, kv, s[5]); s[6] = fmaf(qb.z, kv, s[6]); s[7] = fmaf(qb.w, kv, s[7]);
          }
        } else {
          for (int c = 0; c < d; ++c) {
            const float kv = krow[c];
            const float4 qa = *reinterpret_cast<const float4*>(myq + c * kWinSlots);
            s[0] = fmaf(qa.x, kv, s[0]); s[1] = fmaf(qa.y, kv, s[1]); s[2] = fmaf(qa.z, kv, s[2]); s[3] = fmaf(qa.w, kv, s[3]);
          }
        }
      }
      const int key = k0 + lane;
      float pw[kWinSlots];
#pragma unroll
      for (int u = 0; u < kWinSlots; ++u) {
        pw[u] = 0.f;
        if (u < ns) {
          const bool vis = lane < n_keys && key <= pos[u] && key >= lo[u];
          float sc = vis ? s[u] - slope[u] * static_cast<float>(pos[u] - key) : -INFINITY;
          if (vis && p.dist_bias != nullptr) sc += p.dist_bias[static_cast<int64_t>(min(pos[u] - key, p.n_bias - 1)) * p.H + hd[u]];
          const float m_new = fmaxf(m[u], warp_max(sc));
          float corr = 1.f;
          if (m_new != -INFINITY) {
            pw[u] = vis ? expf(sc - m_new) : 0.f;
            corr = expf(m[u] - m_new);                    // m = -inf: 0, and l and acc are 0 then
          }
          l[u] = l[u] * corr + warp_sum(pw[u]);
          m[u] = m_new;
#pragma unroll
          for (int k = 0; k < DVR; ++k) acc[u][k] *= corr;
        }
      }
      *reinterpret_cast<float4*>(mysp + lane * kWinSlots) = make_float4(pw[0], pw[1], pw[2], pw[3]);
      *reinterpret_cast<float4*>(mysp + lane * kWinSlots + 4) = make_float4(pw[4], pw[5], pw[6], pw[7]);
      __syncwarp();
      for (int j = 0; j < n_keys; ++j) {
        const float4 pa = *reinterpret_cast<const float4*>(mysp + j * kWinSlots);
        float4 pb = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ns > 4) pb = *reinterpret_cast<const float4*>(mysp + j * kWinSlots + 4);
        const float pj[kWinSlots] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
        for (int k = 0; k < DVR; ++k) {
          const int c = lane + 32 * k;
          if (c < dv) {
            const float vv = sv[j * ldv + c];
#pragma unroll
            for (int u = 0; u < kWinSlots; ++u)
              if (u < 4 || ns > 4) acc[u][k] = fmaf(pj[u], vv, acc[u][k]);
          }
        }
      }
      __syncwarp();
    }
    // write the pairs of this warp
    T* out = static_cast<T*>(p.out);
    const T* gate = static_cast<const T*>(p.gate);
#pragma unroll
    for (int u = 0; u < kWinSlots; ++u) {
      if (u >= ns) continue;
      const int pr = warp + u * NW, qi = pr / n_heads, hh = pr % n_heads, head = g * rep + h_lo + hh;
      const int64_t t = seg + qi;
      float f = p.out_scale / (l[u] > 0.f ? l[u] : 1.f);
      if (gate != nullptr) f *= sigmoidf_(ld(gate + t * p.ldg + head));
#pragma unroll
      for (int k = 0; k < DVR; ++k) {
        const int c = lane + 32 * k;
        if (c < dv) st(out + (t * p.H + head) * dv + c, acc[u][k] * f);
      }
    }
    seg = seg_end;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same attention for a decoding batch (one token per sequence).  grid (tokens, kv heads, head chunks x key splits), four
// warps.  All (at most NP) heads of the chunk share the token, so every warp carries all of them and the warps divide the KEYS:
// of a staged tile of 32 keys warp w owns keys 8 w .. 8 w + 7.  Scores: lane = (key, quarter); a lane walks channels
// quarter, quarter + 4, ... of its key for all heads at once (queries head-interleaved: one vector read per channel), and
// two shuffles add the quarters.  Each warp keeps an online softmax state (m, l, sum) over its own keys; values: a lane
// owns channels lane, lane + 32, ... for all heads.  The four states are merged through shared memory at the end, and go
// to the output or, with key splits, to the workspace of the merge kernel.  The page slots of a tile are looked up one tile
// ahead by 32 threads, so that staging has no divisions.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kDecWarps = 4, kDecKeys = kWinTile / kDecWarps;

template <typename T> struct StageVec;
template <> struct StageVec<float> {
  static constexpr int kN = 4;
  using Raw = float4;
  static __device__ __forceinline__ Raw fetch(const float* src) { return *reinterpret_cast<const float4*>(src); }
  static __device__ __forceinline__ void put(float* o, const Raw& r) { *reinterpret_cast<float4*>(o) = r; }
};
template <> struct StageVec<__nv_bfloat16> {
  static constexpr int kN = 8;
  using Raw = uint4;
  static __device__ __forceinline__ Raw fetch(const __nv_bfloat16* src) { return *reinterpret_cast<const uint4*>(src); }
  static __device__ __forceinline__ void put(float* o, const Raw& r) {
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
    const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]), c = __bfloat1622float2(h2[2]), e = __bfloat1622float2(h2[3]);
    *reinterpret_cast<float4*>(o) = make_float4(a.x, a.y, b.x, b.y);
    *reinterpret_cast<float4*>(o + 4) = make_float4(c.x, c.y, e.x, e.y);
  }
};
// Rows of `width` values at the cached slots `slots[j]`, of one or two caches of equal width, -> dst[j][ld] as fp32 (ld a
// multiple of 4).  Loads go out in batches of kStageBatch per cache before the first dependent store.
constexpr int kStageBatch = 4;
template <typename T, bool kTwo>
__device__ __forceinline__ void stage_slots(float* dst_a, int ld_a, const T* cache_a, float* dst_b, int ld_b, const T* cache_b,
                                            const int64_t* slots, int G, int g, int width, int n_keys) {
  constexpr int V = StageVec<T>::kN;
  using Raw = typename StageVec<T>::Raw;
  if (width % V == 0) {
    const int per_row = width / V, total = n_keys * per_row;
    const int sh = (per_row & (per_row - 1)) == 0 ? __ffs(per_row) - 1 : -1;
    for (int i0 = threadIdx.x; i0 < total; i0 += kStageBatch * blockDim.x) {
      Raw ra[kStageBatch], rb[kStageBatch];
      int off_a[kStageBatch], off_b[kStageBatch];
#pragma unroll
      for (int e = 0; e < kStageBatch; ++e) {
        const int i = i0 + e * blockDim.x;
        off_a[e] = -1;
        if (i < total) {
          const int j = sh >= 0 ? i >> sh : i / per_row, c = (i - j * per_row) * V;
          const int64_t src = (slots[j] * G + g) * width + c;
          ra[e] = StageVec<T>::fetch(cache_a + src);
          if (kTwo) rb[e] = StageVec<T>::fetch(cache_b + src);
          off_a[e] = j * ld_a + c;
          off_b[e] = j * ld_b + c;
        }
      }
#pragma unroll
      for (int e = 0; e < kStageBatch; ++e) {
        if (off_a[e] >= 0) {
          StageVec<T>::put(dst_a + off_a[e], ra[e]);
          if (kTwo) StageVec<T>::put(dst_b + off_b[e], rb[e]);
        }
      }
    }
  } else {
    for (int i = threadIdx.x; i < n_keys * width; i += blockDim.x) {
      const int j = i / width, c = i - j * width;
      const int64_t src = (slots[j] * G + g) * width + c;
      dst_a[j * ld_a + c] = ld(cache_a + src);
      if (kTwo) dst_b[j * ld_b + c] = ld(cache_b + src);
    }
  }
}

template <typename T, int DVR, int NP>
__global__ void __launch_bounds__(kDecWarps * 32, 4) window_attention_decode_kernel(WindowAttnArgs p) {
  extern __shared__ __align__(16) float smem[];
  const int d = p.d, dv = p.dv;
  const int dq = (d + 3) / 4 * 4, ldk = dq + 4, ldv = (dv + 3) / 4 * 4;   // ldk = 4 mod 32 for d a multiple of 32: no bank conflicts
  float* sq = smem;                                        // [d][NP]
  float* sk = sq + dq * NP;                                // [tile][ldk]
  float* sv = sk + kWinTile * ldk;                         // [tile][ldv]
  int64_t* sslot = reinterpret_cast<int64_t*>(sv + kWinTile * ldv);       // [2][tile]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, kl = lane >> 2, part = lane & 3;
  const int t = blockIdx.x, g = blockIdx.y, rep = p.H / p.G;
  const int chunk = blockIdx.z / p.n_splits, split = blockIdx.z % p.n_splits;
  const int h_lo = chunk * p.HC, n_heads = min(p.HC, rep - h_lo);
  const T* kc = static_cast<const T*>(p.kcache);
  const T* vc = static_cast<const T*>(p.vcache);
  const int* table = p.block_table + static_cast<int64_t>(p.tok_req[t]) * p.max_blocks;
  const int pos = p.tok_len[t] - 1;
  const int lo = p.window > 0 ? max(0, pos + 1 - p.window) : 0;
  int k_begin = lo, k_end = pos + 1;
  if (p.n_splits > 1) {                                    // the visible keys are cut into n_splits runs of whole tiles
    const int per = ((k_end - k_begin + p.n_splits - 1) / p.n_splits + kWinTile - 1) / kWinTile * kWinTile;
    k_begin += split * per;
    k_end = min(k_end, k_begin + per);
  }
  const T* qrow = static_cast<const T*>(p.q) + static_cast<int64_t>(t) * p.ldq + static_cast<int64_t>(g * rep + h_lo) * d;
  for (int i = threadIdx.x; i < d * NP; i += blockDim.x) {
    const int c = i / NP, u = i % NP;
    sq[i] = u < n_heads ? ld(qrow + u * d + c) * p.scale : 0.f;
  }
  auto slot_of = [&](int key) {
    return static_cast<int64_t>(table[key / p.block_size]) * p.block_size + key % p.block_size;
  };
  if (threadIdx.x < kWinTile && k_begin + static_cast<int>(threadIdx.x) < k_end) sslot[threadIdx.x] = slot_of(k_begin + threadIdx.x);

  float m[NP], l[NP], slope[NP], acc[NP][DVR];
  const bool with_sink = p.sink && split == 0 && warp == 0;
#pragma unroll
  for (int u = 0; u < NP; ++u) {
    m[u] = with_sink ? 0.f : -INFINITY;
    l[u] = with_sink ? 1.f : 0.f;
    slope[u] = (p.slopes != nullptr && u < n_heads) ? p.slopes[g * rep + h_lo + u] : 0.f;
#pragma unroll
    for (int k = 0; k < DVR; ++k) acc[u][k] = 0.f;
  }
  int it = 0;
  for (int k0 = k_begin; k0 < k_end; k0 += kWinTile, ++it) {
    const int n_keys = min(kWinTile, k_end - k0);
    __syncthreads();                                       // the previous tile is used up; sq and this tile's slots are written
    const int64_t* slots = sslot + (it & 1) * kWinTile;
    if (threadIdx.x < kWinTile && k0 + kWinTile + static_cast<int>(threadIdx.x) < k_end)
      sslot[((it + 1) & 1) * kWinTile + threadIdx.x] = slot_of(k0 + kWinTile + threadIdx.x);
    if (d == dv) {
      stage_slots<T, true>(sk, ldk, kc, sv, ldv, vc, slots, p.G, g, d, n_keys);
    } else {
      stage_slots<T, false>(sk, ldk, kc, nullptr, 0, nullptr, slots, p.G, g, d, n_keys);
      stage_slots<T, false>(sv, ldv, vc, nullptr, 0, nullptr, slots, p.G, g, dv, n_keys);
    }
    __syncthreads();
    const int row0 = warp * kDecKeys;
    if (row0 >= n_keys) continue;                          // none of this warp's keys in the last tile
    const int row = row0 + kl, key = k0 + row;
    const bool vis = row < n_keys;                         // k_begin >= lo and k_end <= pos + 1: every staged key is visible
    float s[NP];
#pragma unroll
    for (int u = 0; u < NP; ++u) s[u] = 0.f;
    if (vis) {
      const float* krow = sk + row * ldk;
      for (int c = part; c < d; c += 4) {
        const float kv = krow[c];
        const float* qc = sq + c * NP;
        if constexpr (NP % 4 == 0) {
#pragma unroll
          for (int v = 0; v < NP / 4; ++v) {
            const float4 qa = *reinterpret_cast<const float4*>(qc + 4 * v);
            s[4 * v] = fmaf(qa.x, kv, s[4 * v]); s[4 * v + 1] = fmaf(qa.y, kv, s[4 * v + 1]);
            s[4 * v + 2] = fmaf(qa.z, kv, s[4 * v + 2]); s[4 * v + 3] = fmaf(qa.w, kv, s[4 * v + 3]);
          }
        } else if constexpr (NP == 2) {
          const float2 qa = *reinterpret_cast<const float2*>(qc);
          s[0] = fmaf(qa.x, kv, s[0]); s[1] = fmaf(qa.y, kv, s[1]);
        } else {
          s[0] = fmaf(qc[0], kv, s[0]);
        }
      }
    }
    float pw[NP];
    const float dist = static_cast<float>(pos - key);
    const float* brow = (p.dist_bias != nullptr && vis) ? p.dist_bias + static_cast<int64_t>(min(pos - key, p.n_bias - 1)) * p.H + g * rep + h_lo
                                                        : nullptr;
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      pw[u] = 0.f;
      if (u < n_heads) {
        float su = s[u];
        su += __shfl_xor_sync(0xffffffffu, su, 1);
        su += __shfl_xor_sync(0xffffffffu, su, 2);
        float sc = vis ? su - slope[u] * dist : -INFINITY;
        if (brow != nullptr) sc += brow[u];
        const float m_new = fmaxf(m[u], warp_max(sc));     // finite: the warp's first key is visible
        pw[u] = vis ? expf(sc - m_new) : 0.f;
        const float corr = expf(m[u] - m_new);             // m = -inf: 0, and l and acc are 0 then
        l[u] = l[u] * corr + warp_sum(part == 0 ? pw[u] : 0.f);
        m[u] = m_new;
#pragma unroll
        for (int k = 0; k < DVR; ++k) acc[u][k] *= corr;
      }
    }
    const int mine = min(kDecKeys, n_keys - row0);
    for (int jj = 0; jj < mine; ++jj) {
      float pj[NP];
#pragma unroll
      for (int u = 0; u < NP; ++u) pj[u] = __shfl_sync(0xffffffffu, pw[u], jj * 4);
      const float* vrow = sv + (row0 + jj) * ldv;
#pragma unroll
      for (int k = 0; k < DVR; ++k) {
        const int c = lane + 32 * k;
        if (c < dv) {
          const float vv = vrow[c];
#pragma unroll
          for (int u = 0; u < NP; ++u) acc[u][k] = fmaf(pj[u], vv, acc[u][k]);
        }
      }
    }
  }
  // merge the four warps' states: [warp][head][m, l, sum(dv)] over the tile buffers
  __syncthreads();
  float* sm = sk;
  const int ldm = dv + 2;
#pragma unroll
  for (int u = 0; u < NP; ++u) {
    if (u >= n_heads) continue;
    float* w = sm + (warp * NP + u) * ldm;
    if (lane == 0) { w[0] = m[u]; w[1] = l[u]; }
#pragma unroll
    for (int k = 0; k < DVR; ++k) {
      const int c = lane + 32 * k;
      if (c < dv) w[2 + c] = acc[u][k];
    }
  }
  __syncthreads();
  for (int u = warp; u < n_heads; u += kDecWarps) {
    float M = -INFINITY, f[kDecWarps], L = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) M = fmaxf(M, sm[(w * NP + u) * ldm]);
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float mw = sm[(w * NP + u) * ldm];
      f[w] = (mw != -INFINITY) ? expf(mw - M) : 0.f;
      L = fmaf(sm[(w * NP + u) * ldm + 1], f[w], L);
    }
    const int head = g * rep + h_lo + u;
    const int64_t orow = static_cast<int64_t>(t) * p.H + head;
    float* wsrow = p.n_splits > 1 ? p.ws + (orow * p.n_splits + split) * ldm : nullptr;
    float fo = 0.f;
    if (wsrow != nullptr) {
      if (lane == 0) { wsrow[0] = M; wsrow[1] = L; }
    } else {
      fo = p.out_scale / (L > 0.f ? L : 1.f);
      if (p.gate != nullptr) fo *= sigmoidf_(ld(static_cast<const T*>(p.gate) + static_cast<int64_t>(t) * p.ldg + head));
    }
    for (int c = lane; c < dv; c += 32) {
      float a = 0.f;
#pragma unroll
      for (int w = 0; w < kDecWarps; ++w) a = fmaf(sm[(w * NP + u) * ldm + 2 + c], f[w], a);
      if (wsrow != nullptr) wsrow[2 + c] = a;
      else st(static_cast<T*>(p.out) + orow * dv + c, a * fo);
    }
  }
}

// one warp per (token, head): the partial results of the key splits become the head's output
template <typename T>
__global__ void __launch_bounds__(128) window_attention_merge_kernel(WindowAttnArgs p) {
  const int64_t row = static_cast<int64_t>(blockIdx.x) * 4 + (threadIdx.x >> 5);
  if (row >= static_cast<int64_t>(p.n_tok) * p.H) return;
  const int lane = threadIdx.x & 31, dv = p.dv;
  const int64_t t = row / p.H;
  const int head = static_cast<int>(row % p.H);
  const int ldm = dv + 2;
  const float* w = p.ws + row * p.n_splits * ldm;
  // the weights of the (at most 64) splits: lane s holds those of splits s and s + 32
  const bool has0 = lane < p.n_splits, has1 = lane + 32 < p.n_splits;
  const float m0 = has0 ? w[lane * ldm] : -INFINITY, m1 = has1 ? w[(lane + 32) * ldm] : -INFINITY;
  const float l0 = has0 ? w[lane * ldm + 1] : 0.f, l1 = has1 ? w[(lane + 32) * ldm + 1] : 0.f;
  const float M = warp_max(fmaxf(m0, m1));
  const float f0 = m0 != -INFINITY ? expf(m0 - M) : 0.f, f1 = m1 != -INFINITY ? expf(m1 - M) : 0.f;
  const float L = warp_sum(l0 * f0 + l1 * f1);
  float f = p.out_scale / (L > 0.f ? L : 1.f);
  if (p.gate != nullptr) f *= sigmoidf_(ld(static_cast<const T*>(p.gate) + t * p.ldg + head));
  for (int c0 = 0; c0 < dv; c0 += 32) {
    const int c = c0 + lane;
    float a = 0.f;
    for (int s = 0; s < p.n_splits; ++s) {
      const float fs = __shfl_sync(0xffffffffu, s < 32 ? f0 : f1, s & 31);
      if (c < dv) a = fmaf(w[s * ldm + 2 + c], fs, a);
    }
    if (c < dv) st(static_cast<T*>(p.out) + row * dv + c, a * f);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Selective scan.  Per channel c and state n:  S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n;  y_c = sum_n S[c, n] C_n +
// D_c x_c, then y * silu(z) * out_scale.  dt = softplus(dt_pre + dt_bias), A = -exp(A_log).
// grid (channel blocks of 32, sequences).  The N states of a channel are spread over 4 adjacent lanes (state n on lane n % 4);
// dt, x, B and C of 16 tokens are staged in shared memory per round, so the sequential part touches registers and shared
// memory only.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kSelThreads = 128, kSelParts = 4, kSelCh = kSelThreads / kSelParts, kSelChunk = 16;

template <typename T, int NS>
__global__ void __launch_bounds__(kSelThreads) selective_scan_kernel(SelScanArgs p) {
  extern __shared__ float smem[];
  const int N = p.N;
  float* sdt = smem;                                 // [chunk][32]
  float* sx = sdt + kSelChunk * kSelCh;              // [chunk][32]
  float* sz = sx + kSelChunk * kSelCh;               // [chunk][32]  silu(z) * out_scale
  float* sy = sz + kSelChunk * kSelCh;               // [chunk][32]  outputs of the round
  float* sB = sy + kSelChunk * kSelCh;               // [chunk][N]
  float* sC = sB + kSelChunk * N;                    // [chunk][N]
  const int r = blockIdx.y, part = threadIdx.x & (kSelParts - 1), cl = threadIdx.x >> 2;
  const int c0 = blockIdx.x * kSelCh, c = c0 + cl;
  const bool live = c < p.C;
  const int a = p.cu[r], b = p.cu[r + 1];
  if (a >= b) return;
  const T* x = static_cast<const T*>(p.x);
  const T* z = static_cast<const T*>(p.z);
  const T* Bm = static_cast<const T*>(p.B);
  const T* Cm = static_cast<const T*>(p.Cm);
  T* y = static_cast<T*>(p.y);
  float A[NS], S[NS];
  float* st_row = p.state + (static_cast<int64_t>(p.rows[r]) * p.C + (live ? c : 0)) * N;
#pragma unroll
  for (int i = 0; i < NS; ++i) {
    const int n = part + kSelParts * i;
    const bool ok = live && n < N;
    // decay exp(dt * A) = 2^(dt * A * log2 e), A = -exp(A_log)
    A[i] = ok ? -expf(ld(static_cast<const T*>(p.A_log) + static_cast<int64_t>(c) * N + n)) * 1.4426950408889634f : 0.f;
    S[i] = ok ? st_row[n] : 0.f;
  }
  const float Dc = live ? ld(static_cast<const T*>(p.D) + c) : 0.f;
  for (int t0 = a; t0 < b; t0 += kSelChunk) {
    const int nt = min(kSelChunk, b - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * kSelCh; i += kSelThreads) {
      const int tt = i / kSelCh, cc = i % kSelCh;
      float dtv = 0.f, xv = 0.f, zg = p.out_scale;
      if (c0 + cc < p.C) {
        if (z != nullptr) { const float zv = ld(z + static_cast<int64_t>(t0 + tt) * p.ldz + c0 + cc); zg *= zv * sigmoidf_(zv); }
        const float pre = p.dt_pre[static_cast<int64_t>(t0 + tt) * p.lddt + c0 + cc] +
                          (p.dt_bias != nullptr ? ld(static_cast<const T*>(p.dt_bias) + c0 + cc) : 0.f);
        dtv = pre > 20.f ? pre : log1pf(expf(pre));
        xv = ld(x + static_cast<int64_t>(t0 + tt) * p.ldx + c0 + cc);
      }
      sdt[i] = dtv; sx[i] = xv; sz[i] = zg;
    }
    for (int i = threadIdx.x; i < nt * N; i += kSelThreads) {
      const int tt = i / N, n = i % N;
      sB[i] = ld(Bm + static_cast<int64_t>(t0 + tt) * p.ldb + n);
      sC[i] = ld(Cm + static_cast<int64_t>(t0 + tt) * p.ldc + n);
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dtv = sdt[tt * kSelCh + cl], xv = sx[tt * kSelCh + cl];
      const float dx = dtv * xv;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NS; ++i) {
        const int n = part + kSelParts * i;
        if (n < N) {
          S[i] = fmaf(exp2f(dtv * A[i]), S[i], dx * sB[tt * N + n]);
          acc = fmaf(S[i], sC[tt * N + n], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (part == 0) sy[tt * kSelCh + cl] = fmaf(Dc, xv, acc) * sz[tt * kSelCh + cl];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nt * kSelCh; i += kSelThreads) {
      const int tt = i / kSelCh, cc = i % kSelCh;
      if (c0 + cc < p.C) st(y + static_cast<int64_t>(t0 + tt) * p.ldy + c0 + cc, sy[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < NS; ++i) {
    const int n = part + kSelParts * i;
    if (live && n < N) st_row[n] = S[i];
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------------
bool stream_mix_norm(const StreamNormArgs& p, int n_tok, bool bf16, cudaStream_t s) {
  if (p.S < 1 || p.S > kMaxStreams) return false;
  if (n_tok == 0) return true;
  const size_t smem = p.inp != nullptr ? static_cast<size_t>(p.W) * sizeof(float) : 0;
  if (smem > 200 * 1024) return false;
  const size_t esz = bf16 ? 2 : 4;
  auto al = [&](const void* q, size_t bytes) { return q == nullptr || reinterpret_cast<uintptr_t>(q) % bytes == 0; };
  const bool vec = p.W % 4 == 0 && p.S <= 4 && al(p.x, 16) && al(p.a, 4 * esz) && al(p.b, 4 * esz) && al(p.bias_a, 4 * esz) &&
                   al(p.ls, 4 * esz) && al(p.w, 4 * esz) && al(p.beta, 4 * esz) && al(p.h, 4 * esz) && p.lda % 4 == 0 && p.ldb % 4 == 0;
#define SEQ_STREAM_VEC(SS)                                                                                                  \
  {                                                                                                                         \
    if (smem > 48 * 1024)                                                                                                   \
      cudaFuncSetAttribute(stream_mix_norm_vec_kernel<T, SS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    stream_mix_norm_vec_kernel<T, SS><<<n_tok, 256, smem, s>>>(p);                                                          \
  }
  SEQ_DISPATCH_T(bf16, {
    if (vec && p.S == 1) SEQ_STREAM_VEC(1)
    else if (vec && p.S == 2) SEQ_STREAM_VEC(2)
    else if (vec && p.S == 3) SEQ_STREAM_VEC(3)
    else if (vec && p.S == 4) SEQ_STREAM_VEC(4)
    else {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(stream_mix_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
      stream_mix_norm_kernel<T><<<n_tok, 256, smem, s>>>(p);
    }
  });
#undef SEQ_STREAM_VEC
  return true;
}

void add_sinusoid(float* x, const int64_t* positions, const float* freq, int n_tok, int width, cudaStream_t s) {
  const int half = width / 2;
  const int64_t n = static_cast<int64_t>(n_tok) * half;
  if (n == 0) return;
  add_sinusoid_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(x, positions, freq, n, half);
}

void head_rms_norm(const void* x, int64_t ldx, const void* w, void* y, int n_tok, int heads, int d, float eps, bool bf16,
                   cudaStream_t s) {
  const int64_t rows = static_cast<int64_t>(n_tok) * heads;
  if (rows == 0) return;
  SEQ_DISPATCH_T(bf16, head_rms_norm_kernel<T><<<static_cast<unsigned>((rows + 3) / 4), 128, 0, s>>>(
                           static_cast<const T*>(x), ldx, static_cast<const T*>(w), static_cast<T*>(y), rows, heads, d, eps));
}

void window_attention_shape(int H, int G, int* QB, int* HC) {
  const int rep = H / G;
  *HC = std::min(rep, kWinWarps * kWinSlots);
  *QB = std::max(1, (kWinWarps * kWinSlots) / *HC);
}

constexpr int kDecMaxHeads = 8;                            // heads of one kv head that a decoding CTA carries

int window_attention_splits(int H, int G, int n_tok, int max_keys) {
  const int rep = H / G, hc = std::min(rep, kDecMaxHeads);
  const int ctas = n_tok * G * ((rep + hc - 1) / hc);
  const int by_keys = (max_keys + 2 * kWinTile - 1) / (2 * kWinTile);     // at least two tiles per split
  const int by_fill = (8 * 148 + ctas - 1) / ctas;
  return std::max(1, std::min(std::min(by_keys, by_fill), 64));
}

template <typename T, int DVR>
static bool launch_window(WindowAttnArgs& p, cudaStream_t s) {
  const int rep = p.H / p.G;
  window_attention_shape(p.H, p.G, &p.QB, &p.HC);
  p.n_splits = 1;
  const size_t smem = (static_cast<size_t>(kWinWarps) * kWinSlots * p.d + static_cast<size_t>(kWinTile) * (p.d + 1) +
                       static_cast<size_t>(kWinTile) * p.dv + static_cast<size_t>(kWinWarps) * kWinSlots * kWinTile) * sizeof(float);
  if (smem > 220 * 1024) return false;
  dim3 grid((p.n_tok + p.QB - 1) / p.QB, p.G, (rep + p.HC - 1) / p.HC);
  if (grid.z > 65535) return false;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(window_attention_kernel<T, DVR>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  window_attention_kernel<T, DVR><<<grid, kWinWarps * 32, smem, s>>>(p);
  return true;
}

template <typename T, int DVR, int NP>
static bool launch_decode(WindowAttnArgs& p, cudaStream_t s) {
  const int rep = p.H / p.G;
  p.QB = 1;
  p.HC = std::min(rep, NP);
  if (p.n_splits < 1) p.n_splits = 1;
  const int dq = (p.d + 3) / 4 * 4, ldv = (p.dv + 3) / 4 * 4;
  const size_t smem = (static_cast<size_t>(dq) * NP + static_cast<size_t>(kWinTile) * (dq + 4) + static_cast<size_t>(kWinTile) * ldv) *
                          sizeof(float) + 2 * kWinTile * sizeof(int64_t);
  if (smem > 220 * 1024) return false;
  dim3 grid(p.n_tok, p.G, ((rep + p.HC - 1) / p.HC) * p.n_splits);
  if (grid.z > 65535) return false;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(window_attention_decode_kernel<T, DVR, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  window_attention_decode_kernel<T, DVR, NP><<<grid, kDecWarps * 32, smem, s>>>(p);
  if (p.n_splits > 1) {
    const int64_t rows = static_cast<int64_t>(p.n_tok) * p.H;
    window_attention_merge_kernel<T><<<static_cast<unsigned>((rows + 3) / 4), 128, 0, s>>>(p);
  }
  return true;
}

template <typename T, int DVR>
static bool launch_decode_heads(WindowAttnArgs& p, cudaStream_t s) {
  const int rep = p.H / p.G;
  if (rep == 1) return launch_decode<T, DVR, 1>(p, s);
  if (rep == 2) return launch_decode<T, DVR, 2>(p, s);
  if (rep <= 4) return launch_decode<T, DVR, 4>(p, s);
  return launch_decode<T, DVR, kDecMaxHeads>(p, s);
}

bool window_attention_paged(const WindowAttnArgs& p_in, bool bf16, cudaStream_t s) {
  WindowAttnArgs p = p_in;
  if (p.n_tok == 0) return true;
  if (p.H % p.G != 0 || p.G > 65535) return false;
  if (p.n_splits > 1 && (p.ws == nullptr || !p.decode)) return false;
  if (p.decode) {
    SEQ_DISPATCH_T(bf16, {
      if (p.dv <= 32) return launch_decode_heads<T, 1>(p, s);
      if (p.dv <= 64) return launch_decode_heads<T, 2>(p, s);
      if (p.dv <= 128) return launch_decode_heads<T, 4>(p, s);
      if (p.dv <= 256) return launch_decode_heads<T, 8>(p, s);
    });
    return false;
  }
  SEQ_DISPATCH_T(bf16, {
    if (p.dv <= 32) return launch_window<T, 1>(p, s);
    if (p.dv <= 64) return launch_window<T, 2>(p, s);
    if (p.dv <= 128) return launch_window<T, 4>(p, s);
    if (p.dv <= 256) return launch_window<T, 8>(p, s);
  });
  return false;
}

template <typename T, int NS>
static void launch_sel(const SelScanArgs& p, int R, cudaStream_t s) {
  const size_t smem = (4 * static_cast<size_t>(kSelChunk) * kSelCh + 2 * static_cast<size_t>(kSelChunk) * p.N) * sizeof(float);
  dim3 grid((p.C + kSelCh - 1) / kSelCh, R);
  selective_scan_kernel<T, NS><<<grid, kSelThreads, smem, s>>>(p);
}

bool selective_scan(const SelScanArgs& p, int R, bool bf16, cudaStream_t s) {
  if (R == 0) return true;
  if (R > 65535) return false;
  SEQ_DISPATCH_T(bf16, {
    if (p.N <= 16) launch_sel<T, 4>(p, R, s);
    else if (p.N <= 32) launch_sel<T, 8>(p, R, s);
    else if (p.N <= 64) launch_sel<T, 16>(p, R, s);
    else if (p.N <= 128) launch_sel<T, 32>(p, R, s);
    else return false;
  });
  return true;
}

}  // namespace b200seq
