// Kernels of the side-by-side (attention + delta memory) and minGRU mixers over a packed token batch (sm_100a):
// output-side RMS norm fused with the fp32 residual addition (optionally of the mean of two normed branches), whole-projection
// q / k norm with partial interleaved rotary positions, paged grouped-query attention whose softmax weights are mixed across
// heads, the generalized delta-rule scan (per-channel decay and removal), the minGRU scan, and the clamped gated activation.
//
// Conventions as in seqmix.cu: activations are `T` (float or __nv_bfloat16); statistics, angles, scores, weights, gates, decays
// and every recurrent state are fp32; `cu[R + 1]` / `rows[R]` describe the packed batch.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
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
  __syncthreads();                                                  // red may still be read from a previous call
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
  return tot;
}

// ---------------------------------------------------------------------------------------------------------------------
// x (fp32, in place) += rms_norm(m) * (w_off + w), y = x in the activation type.  m is `a`, or, with a second branch,
// (rms_norm(a) * wa + rms_norm(b) * wb) / 2.  One CTA per token.
// ---------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) norm_add_kernel(float* __restrict__ x, const T* __restrict__ a, const T* __restrict__ b,
                                                       const T* __restrict__ wa, const T* __restrict__ wb, const T* __restrict__ w,
                                                       T* __restrict__ y, int cols, float eps, float w_off,
                                                       const T* __restrict__ extra, const T* __restrict__ next_w) {
  extern __shared__ float row[];
  __shared__ float red[32];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * cols;
  const float inv_n = 1.0f / static_cast<float>(cols);
  if (b != nullptr) {
    float sa = 0.f, sb = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
      const float va = ld(a + base + c), vb = ld(b + base + c);
      sa += va * va; sb += vb * vb;
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, red) * inv_n + eps);
    const float rb = 1.0f / sqrtf(block_sum(sb, red) * inv_n + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x)
      row[c] = 0.5f * (ld(a + base + c) * ra * ld(wa + c) + ld(b + base + c) * rb * ld(wb + c));
  } else {
    for (int c = threadIdx.x; c < cols; c += blockDim.x) row[c] = ld(a + base + c);
  }
  float r = 1.f;
  if (w != nullptr) {
    float ss = 0.f;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) ss += row[c] * row[c];   // each thread re-reads its own entries
    r = 1.0f / sqrtf(block_sum(ss, red) * inv_n + eps);
  }
  float sx = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float m = w != nullptr ? row[c] * r * (w_off + ld(w + c)) : row[c];
    if (extra != nullptr) m += ld(extra + base + c);
    const float v = x[base + c] + m;
    x[base + c] = v;
    if (next_w != nullptr) { row[c] = v; sx += v * v; }
    else st(y + base + c, v);
  }
  if (next_w != nullptr) {
    const float rx = 1.0f / sqrtf(block_sum(sx, red) * inv_n + eps);
    for (int c = threadIdx.x; c < cols; c += blockDim.x) st(y + base + c, row[c] * rx * ld(next_w + c));
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// q and k of a token: one RMS norm across all heads' channels, with a weight per channel, then rotation of the
// first `rot` dimensions of every head, pairs (2i, 2i + 1), by angle position * inv_freq[i].  grid (tokens, 2): y = 0 is q.
// ---------------------------------------------------------------------------------------------------------------------
template <typename T> struct Pair;
template <> struct Pair<float> {
  static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
  static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <> struct Pair<__nv_bfloat16> {
  static __device__ __forceinline__ float2 load(const __nv_bfloat16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float2 v) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
  }
};

// PAIRED: even head width and strides, bases aligned for two-element accesses (the launcher checks); otherwise element by element.
// The rot / 2 angles of a token are the same for all heads: cosine and sine are made once per CTA.
template <typename T, bool PAIRED>
__global__ void __launch_bounds__(256) norm_rope_kernel(NormRopeArgs p) {
  extern __shared__ float row[];                                    // [n] values, then [rot] cosines and sines
  __shared__ float red[32];
  const int t = blockIdx.x, which = blockIdx.y;
  const int n = which == 0 ? p.q_ch : p.k_ch;
  const T* src = static_cast<const T*>(which == 0 ? p.q : p.k) + static_cast<int64_t>(t) * (which == 0 ? p.ldq : p.ldk);
  const T* w = static_cast<const T*>(which == 0 ? p.wq : p.wk);
  T* dst = static_cast<T*>(which == 0 ? p.q_out : p.k_out) + static_cast<int64_t>(t) * n;
  float* cs = row + n + (n & 1);
  const int half = p.rot / 2;
  float ss = 0.f;
  constexpr int NP = 4;                                             // pairs a thread keeps in registers
  const bool in_regs = PAIRED && n <= 2 * NP * 256;
  float2 held[NP];
  if (in_regs) {
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      const int c = 2 * (threadIdx.x + u * 256);
      held[u] = c < n ? Pair<T>::load(src + c) : make_float2(0.f, 0.f);
      ss += held[u].x * held[u].x + held[u].y * held[u].y;
    }
  } else if (PAIRED) {
    for (int c = 2 * threadIdx.x; c < n; c += 2 * blockDim.x) {
      const float2 v = Pair<T>::load(src + c);
      row[c] = v.x; row[c + 1] = v.y;
      ss += v.x * v.x + v.y * v.y;
    }
  } else {
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      const float v = ld(src + c);
      row[c] = v;
      ss += v * v;
    }
  }
  if (threadIdx.x < half) {
    const float ang = static_cast<float>(p.positions[t]) * p.inv_freq[threadIdx.x];
    cs[2 * threadIdx.x] = cosf(ang);
    cs[2 * threadIdx.x + 1] = sinf(ang);
  }
  for (int i = threadIdx.x + blockDim.x; i < half; i += blockDim.x) {   // more than 256 rotated pairs per head
    const float ang = static_cast<float>(p.positions[t]) * p.inv_freq[i];
    cs[2 * i] = cosf(ang);
    cs[2 * i + 1] = sinf(ang);
  }
  const float r = 1.0f / sqrtf(block_sum(ss, red) / static_cast<float>(n) + p.eps);   // its barriers also publish row and cs
  const int pairs = p.head_dim / 2, odd = p.head_dim & 1;
  if (in_regs) {
#pragma unroll
    for (int u = 0; u < NP; ++u) {
      const int c = 2 * (threadIdx.x + u * 256);
      if (c >= n) break;
      const int i = (c % p.head_dim) >> 1;
      const float2 wv = Pair<T>::load(w + c);
      float a0 = held[u].x * r * wv.x, a1 = held[u].y * r * wv.y;
      if (i < half) {
        const float c_ = cs[2 * i], s_ = cs[2 * i + 1];
        const float b0 = a0 * c_ - a1 * s_, b1 = a1 * c_ + a0 * s_;
        a0 = b0; a1 = b1;
      }
      Pair<T>::store(dst + c, make_float2(a0, a1));
    }
    return;
  }
  for (int e = threadIdx.x; e < (n / p.head_dim) * (pairs + odd); e += blockDim.x) {
    const int h = e / (pairs + odd), i = e % (pairs + odd);
    const int c = h * p.head_dim + 2 * i;
    if (i >= pairs) { st(dst + c, row[c] * r * ld(w + c)); continue; }   // the last channel of an odd head width
    float2 wv;
    if (PAIRED) wv = Pair<T>::load(w + c);
    else wv = make_float2(ld(w + c), ld(w + c + 1));
    float u = row[c] * r * wv.x, v = row[c + 1] * r * wv.y;
    if (i < half) {
      const float c_ = cs[2 * i], s_ = cs[2 * i + 1];
      const float u2 = u * c_ - v * s_, v2 = v * c_ + u * s_;
      u = u2; v = v2;
    }
    if (PAIRED) Pair<T>::store(dst + c, make_float2(u, v));
    else { st(dst + c, u); st(dst + c + 1, v); }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// Paged grouped-query attention with head mixing.  Per query token i and head h:
//   P_g(i, j) = softmax_j(q_g . k_kv(g)(j) * scale)  over the visible keys;  M_h = sum_g talk[h, g] P_g;  o_h = sum_j M_h(j) v_kv(h)(j)
// The mixed weights need every head's normaliser, so the keys are walked twice: first for the running maxima and sums of all
// heads, then again for the weights, their mixture and the weighted values (scores are recomputed, bit for bit the same).
// grid (tokens, key splits).  MODE 0: one split, both walks, output written.  MODE 1: first walk of a split -> (max, sum) per
// head in the workspace.  MODE 2: second walk of a split with the merged statistics -> partial sums in the workspace (a merge
// kernel adds them up).  Keys and values of a tile of `key_tile` tokens are staged in shared memory.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kMixThreads = 256;

template <typename T, int NACC, int MODE>
__global__ void __launch_bounds__(kMixThreads) mixed_attention_kernel(MixAttnArgs p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, G = p.G, d = p.d, dv = p.dv, KT = p.key_tile, rep = H / G;
  const int ldk = p.ldk_s, ldv = G * dv;
  float* sq = reinterpret_cast<float*>(smem_raw);                  // [H * d]
  float* sS = sq + H * d;                                          // [H * KT] scores, then weights
  float* sP = sS + H * KT;                                         // [H * KT] mixed weights
  float* sT = sP + H * KT;                                         // [H * H]
  float* sm = sT + H * H;                                          // [H]
  float* sl = sm + H;                                              // [H]
  int* sslot = reinterpret_cast<int*>(sl + H);                     // [KT]
  // the fp32 / int part above is padded by the host to a multiple of 4 words (p.head_words), so the tiles stay 16-byte aligned
  T* sK = reinterpret_cast<T*>(smem_raw + static_cast<size_t>(p.head_words) * 4);
  T* sV = sK + static_cast<size_t>(KT) * ldk;
  const int t = blockIdx.x, z = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = kMixThreads >> 5;
  const int len = p.tok_len[t];
  const int per_split = (len + p.n_splits - 1) / p.n_splits;
  const int key_lo = z * per_split, key_hi = min(len, key_lo + per_split);
  const int* table = p.block_table + static_cast<int64_t>(p.tok_req[t]) * p.max_blocks;
  const T* kc = static_cast<const T*>(p.kcache);
  const T* vc = static_cast<const T*>(p.vcache);
  const T* q = static_cast<const T*>(p.q) + static_cast<int64_t>(t) * p.ldq;
  for (int e = threadIdx.x; e < H * d; e += kMixThreads) sq[e] = ld(q + e) * p.scale;
  for (int e = threadIdx.x; e < H * H; e += kMixThreads) sT[e] = p.talk != nullptr ? p.talk[e] : ((e / H) == (e % H) ? 1.f : 0.f);
  if (MODE == 2) {                                                 // merge the splits' statistics
    for (int g = warp; g < H; g += n_warps) {
      const float* ws = p.ws_stats + (static_cast<int64_t>(t) * p.n_splits * H + g) * 2;
      float m = -INFINITY;
      for (int s = lane; s < p.n_splits; s += 32) m = fmaxf(m, ws[static_cast<int64_t>(s) * H * 2]);
      m = warp_max(m);
      float l = 0.f;
      for (int s = lane; s < p.n_splits; s += 32) {
        const float ms = ws[static_cast<int64_t>(s) * H * 2];
        if (ms != -INFINITY) l += ws[static_cast<int64_t>(s) * H * 2 + 1] * expf(ms - m);
      }
      l = warp_sum(l);
      if (lane == 0) { sm[g] = m; sl[g] = l; }
    }
  } else {
    for (int g = threadIdx.x; g < H; g += kMixThreads) { sm[g] = -INFINITY; sl[g] = 0.f; }
  }
  float acc[NACC];
#pragma unroll
  for (int n = 0; n < NACC; ++n) acc[n] = 0.f;

  for (int pass = (MODE == 2 ? 1 : 0); pass < (MODE == 1 ? 1 : 2); ++pass) {
    for (int lo = key_lo; lo < key_hi; lo += KT) {
      const int nk = min(KT, key_hi - lo);
      __syncthreads();                                             // the previous tile has been consumed; sq / sT / sm are set
      for (int j = threadIdx.x; j < nk; j += kMixThreads) {
        const int key = lo + j;
        sslot[j] = table[key / p.block_size] * p.block_size + key % p.block_size;
      }
      __syncthreads();
      for (int e = threadIdx.x; e < nk * G * d; e += kMixThreads) {
        const int j = e / (G * d), c = e % (G * d);
        sK[static_cast<size_t>(j) * ldk + c] = kc[static_cast<int64_t>(sslot[j]) * G * d + c];
      }
      if (pass == 1) {
        for (int e = threadIdx.x; e < nk * ldv; e += kMixThreads) {
          const int j = e / ldv, c = e % ldv;
          sV[static_cast<size_t>(j) * ldv + c] = vc[static_cast<int64_t>(sslot[j]) * ldv + c];
        }
      }
      __syncthreads();
      for (int e = threadIdx.x; e < H * KT; e += kMixThreads) {    // scores: a thread per (head, key)
        const int g = e / KT, j = e % KT;
        float s = -INFINITY;
        if (j < nk) {
          const float* qq = sq + g * d;
          const T* kk = sK + static_cast<size_t>(j) * ldk + (g / rep) * d;
          float s0 = 0.f, s1 = 0.f;
          int i = 0;
          for (; i + 1 < d; i += 2) { s0 = fmaf(qq[i], ld(kk + i), s0); s1 = fmaf(qq[i + 1], ld(kk + i + 1), s1); }
          if (i < d) s0 = fmaf(qq[i], ld(kk + i), s0);
          s = s0 + s1;
        }
        sS[e] = s;
      }
      __syncthreads();
      if (pass == 0) {
        for (int g = warp; g < H; g += n_warps) {                  // running maximum and sum of every head
          float mx = -INFINITY;
          for (int j = lane; j < nk; j += 32) mx = fmaxf(mx, sS[g * KT + j]);
          mx = warp_max(mx);
          const float m_old = sm[g], m_new = fmaxf(m_old, mx);
          float sum = 0.f;
          for (int j = lane; j < nk; j += 32) sum += expf(sS[g * KT + j] - m_new);
          sum = warp_sum(sum);
          if (lane == 0) {
            sl[g] = (m_old == -INFINITY ? 0.f : sl[g] * expf(m_old - m_new)) + sum;
            sm[g] = m_new;
          }
        }
        continue;
      }
      for (int e = threadIdx.x; e < H * KT; e += kMixThreads) {    // weights
        const int g = e / KT, j = e % KT;
        sS[e] = j < nk ? expf(sS[e] - sm[g]) / sl[g] : 0.f;
      }
      __syncthreads();
      for (int e = threadIdx.x; e < H * KT; e += kMixThreads) {    // mixture across heads
        const int h = e / KT, j = e % KT;
        float m = 0.f;
        for (int g = 0; g < H; ++g) m = fmaf(sT[h * H + g], sS[g * KT + j], m);
        sP[e] = m;
      }
      __syncthreads();
#pragma unroll
      for (int n = 0; n < NACC; ++n) {                             // weighted values: a thread per (head, value channel)
        const int e = threadIdx.x + n * kMixThreads;
        if (e < H * dv) {
          const int h = e / dv, c = e % dv;
          const float* pw = sP + h * KT;
          const T* vv = sV + (h / rep) * dv + c;
          float a0 = 0.f, a1 = 0.f;
          int j = 0;
          for (; j + 1 < nk; j += 2) {
            a0 = fmaf(pw[j], ld(vv + static_cast<size_t>(j) * ldv), a0);
            a1 = fmaf(pw[j + 1], ld(vv + static_cast<size_t>(j + 1) * ldv), a1);
          }
          if (j < nk) a0 = fmaf(pw[j], ld(vv + static_cast<size_t>(j) * ldv), a0);
          acc[n] += a0 + a1;
        }
      }
    }
  }
  if (MODE == 1) {
    __syncthreads();
    for (int g = threadIdx.x; g < H; g += kMixThreads) {
      float* ws = p.ws_stats + ((static_cast<int64_t>(t) * p.n_splits + z) * H + g) * 2;
      ws[0] = sm[g]; ws[1] = sl[g];
    }
    return;
  }
#pragma unroll
  for (int n = 0; n < NACC; ++n) {
    const int e = threadIdx.x + n * kMixThreads;
    if (e >= H * dv) continue;
    if (MODE == 2) {
      p.ws_acc[(static_cast<int64_t>(t) * p.n_splits + z) * H * dv + e] = acc[n];
    } else {
      float v = acc[n];
      if (p.gate != nullptr) v *= sigmoidf_(ld(static_cast<const T*>(p.gate) + static_cast<int64_t>(t) * p.ldg + e));
      st(static_cast<T*>(p.out) + static_cast<int64_t>(t) * H * dv + e, v);
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// The same attention for head sizes that 16-byte vectors divide (d and dv multiples of 8 for 16-bit, 4 for fp32 activations):
// a CTA serves up to QB consecutive query tokens of one sequence with the same key tile (a block that straddles two sequences
// walks them one after the other); key rows are copied and read 16 bytes at a time (rows padded to 128 m + 16 bytes, so a
// quarter warp's rows fall into distinct banks); a thread owns one (query, key/value head, pair of keys) and keeps the two key
// chunks in registers for the heads of the group; values are not staged: in the weighted sum a thread owns 16 bytes of value channels of
// one head and reads them from the cache once per key for all QB queries.  grid (token blocks, key splits), modes as above.
// ---------------------------------------------------------------------------------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int W = 4;
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* o) { *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]); }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int W = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    o[0] = __uint_as_float(v.x << 16); o[1] = __uint_as_float(v.x & 0xffff0000u);
    o[2] = __uint_as_float(v.y << 16); o[3] = __uint_as_float(v.y & 0xffff0000u);
    o[4] = __uint_as_float(v.z << 16); o[5] = __uint_as_float(v.z & 0xffff0000u);
    o[6] = __uint_as_float(v.w << 16); o[7] = __uint_as_float(v.w & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* o) {
    __nv_bfloat162 a = __floats2bfloat162_rn(o[0], o[1]), b = __floats2bfloat162_rn(o[2], o[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(o[4], o[5]), d = __floats2bfloat162_rn(o[6], o[7]);
    uint4 v;
    v.x = *reinterpret_cast<unsigned*>(&a); v.y = *reinterpret_cast<unsigned*>(&b);
    v.z = *reinterpret_cast<unsigned*>(&c); v.w = *reinterpret_cast<unsigned*>(&d);
    *reinterpret_cast<uint4*>(p) = v;
  }
};

constexpr int kHeadChunk = 4;

template <typename T, int NI, int QB, int MODE>
__global__ void __launch_bounds__(kMixThreads) mixed_attention_vec_kernel(MixAttnArgs p, int n_tok) {
  constexpr int VW = Vec16<T>::W;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int H = p.H, G = p.G, d = p.d, dv = p.dv, KT = p.key_tile, rep = H / G, ldk = p.ldk_s;
  float* sq = reinterpret_cast<float*>(smem_raw);                  // [QB][H * d]
  float* sS = sq + QB * H * d;                                     // [QB][H][KT]
  float* sP = sS + QB * H * KT;                                    // [QB][H][KT]
  float* sT = sP + QB * H * KT;                                    // [H * H]
  float* sm = sT + H * H;                                          // [QB][H]
  float* sl = sm + QB * H;                                         // [QB][H]
  int* sslot = reinterpret_cast<int*>(sl + QB * H);                // [KT]
  int* slen = sslot + KT;                                          // [QB]
  T* sK = reinterpret_cast<T*>(smem_raw + static_cast<size_t>(p.head_words) * 4);
  const int t_lo = blockIdx.x * QB, t_hi = min(n_tok, t_lo + QB), z = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = kMixThreads >> 5;
  const T* kc = static_cast<const T*>(p.kcache);
  const T* vc = static_cast<const T*>(p.vcache);
  const int n_out = H * dv / VW, dvc = dv / VW, krow = G * d / VW;
  for (int e = threadIdx.x; e < H * H; e += kMixThreads) sT[e] = p.talk != nullptr ? p.talk[e] : ((e / H) == (e % H) ? 1.f : 0.f);
  for (int seg_lo = t_lo; seg_lo < t_hi;) {
    const int req = p.tok_req[seg_lo];
    int seg_hi = seg_lo + 1;
    while (seg_hi < t_hi && p.tok_req[seg_hi] == req) ++seg_hi;
    const int nq = seg_hi - seg_lo;
    const int* table = p.block_table + static_cast<int64_t>(req) * p.max_blocks;
    __syncthreads();                                               // the previous segment is done with shared memory
    for (int e = threadIdx.x; e < nq * H * d; e += kMixThreads)
      sq[e] = ld(static_cast<const T*>(p.q) + static_cast<int64_t>(seg_lo + e / (H * d)) * p.ldq + e % (H * d)) * p.scale;
    if (threadIdx.x < nq) slen[threadIdx.x] = p.tok_len[seg_lo + threadIdx.x];
    if (MODE == 2) {
      for (int e = warp; e < nq * H; e += n_warps) {               // merge the splits' statistics of (query, head) e
        const float* ws = p.ws_stats + (static_cast<int64_t>(seg_lo + e / H) * p.n_splits * H + e % H) * 2;
        float m = -INFINITY;
        for (int s = lane; s < p.n_splits; s += 32) m = fmaxf(m, ws[static_cast<int64_t>(s) * H * 2]);
        m = warp_max(m);
        float l = 0.f;
        for (int s = lane; s < p.n_splits; s += 32) {
          const float ms = ws[static_cast<int64_t>(s) * H * 2];
          if (ms != -INFINITY) l += ws[static_cast<int64_t>(s) * H * 2 + 1] * expf(ms - m);
        }
        l = warp_sum(l);
        if (lane == 0) { sm[e] = m; sl[e] = l; }
      }
    } else {
      for (int e = threadIdx.x; e < nq * H; e += kMixThreads) { sm[e] = -INFINITY; sl[e] = 0.f; }
    }
    const int max_len = p.tok_len[seg_hi - 1];                     // visible lengths grow along a sequence's tokens
    const int per_split = (max_len + p.n_splits - 1) / p.n_splits;
    const int key_lo = z * per_split, key_hi = min(max_len, key_lo + per_split);
    float acc[NI][QB][VW];
#pragma unroll
    for (int n = 0; n < NI; ++n)
#pragma unroll
      for (int qi = 0; qi < QB; ++qi)
#pragma unroll
        for (int c = 0; c < VW; ++c) acc[n][qi][c] = 0.f;

    for (int pass = (MODE == 2 ? 1 : 0); pass < (MODE == 1 ? 1 : 2); ++pass) {
      for (int lo = key_lo; lo < key_hi; lo += KT) {
        const int nk = min(KT, key_hi - lo);
        __syncthreads();
        for (int j = threadIdx.x; j < nk; j += kMixThreads) {
          const int key = lo + j;
          sslot[j] = table[key / p.block_size] * p.block_size + key % p.block_size;
        }
        __syncthreads();
        for (int e = threadIdx.x; e < nk * krow; e += kMixThreads) {
          const int j = e / krow, c = e % krow;
          *reinterpret_cast<uint4*>(sK + static_cast<size_t>(j) * ldk + c * VW) =
              *reinterpret_cast<const uint4*>(kc + static_cast<int64_t>(sslot[j]) * G * d + c * VW);
        }
        __syncthreads();
        // scores: a thread per (query, key/value head, pair of keys KT / 2 apart); the query values it reads from shared memory
        // serve both keys and the key chunks stay in registers for the heads of the group
        const int KH = KT / 2;
        for (int e = threadIdx.x; e < nq * G * KH; e += kMixThreads) {
          const int ja = e % KH, jb = ja + KH, c = (e / KH) % G, qi = e / (KH * G);
          const bool va = ja < nk && lo + ja < slen[qi], vb = jb < nk && lo + jb < slen[qi];
          const T* ka = sK + static_cast<size_t>(ja) * ldk + c * d;
          const T* kb = sK + static_cast<size_t>(jb) * ldk + c * d;
          for (int hc = 0; hc < rep; hc += kHeadChunk) {
            float sa[kHeadChunk], sb[kHeadChunk];
#pragma unroll
            for (int r = 0; r < kHeadChunk; ++r) sa[r] = sb[r] = 0.f;
            if (va) {                                              // vb implies va: visibility ends at one key
              const float* qq = sq + (qi * H + c * rep + hc) * d;
              for (int i = 0; i < d; i += VW) {
                float kva[VW], kvb[VW];
                Vec16<T>::load(ka + i, kva);
                Vec16<T>::load(kb + i, kvb);                       // a row past the tile's end holds stale, unused data
#pragma unroll
                for (int r = 0; r < kHeadChunk; ++r) {
                  if (hc + r < rep) {
#pragma unroll
                    for (int u = 0; u < VW; u += 4) {
                      const float4 qv = *reinterpret_cast<const float4*>(qq + r * d + i + u);
                      sa[r] = fmaf(qv.x, kva[u], sa[r]); sb[r] = fmaf(qv.x, kvb[u], sb[r]);
                      sa[r] = fmaf(qv.y, kva[u + 1], sa[r]); sb[r] = fmaf(qv.y, kvb[u + 1], sb[r]);
                      sa[r] = fmaf(qv.z, kva[u + 2], sa[r]); sb[r] = fmaf(qv.z, kvb[u + 2], sb[r]);
                      sa[r] = fmaf(qv.w, kva[u + 3], sa[r]); sb[r] = fmaf(qv.w, kvb[u + 3], sb[r]);
                    }
                  }
                }
              }
            }
#pragma unroll
            for (int r = 0; r < kHeadChunk; ++r) {
              if (hc + r < rep) {
                float* dst = sS + (qi * H + c * rep + hc + r) * KT;
                dst[ja] = va ? sa[r] : -INFINITY;
                dst[jb] = vb ? sb[r] : -INFINITY;
              }
            }
          }
        }
        __syncthreads();
        if (pass == 0) {
          for (int e = warp; e < nq * H; e += n_warps) {           // running maximum and sum of every (query, head)
            float mx = -INFINITY;
            for (int j = lane; j < nk; j += 32) mx = fmaxf(mx, sS[e * KT + j]);
            mx = warp_max(mx);
            if (mx == -INFINITY) continue;                         // nothing of this tile is visible to the query
            const float m_old = sm[e], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (int j = lane; j < nk; j += 32) sum += expf(sS[e * KT + j] - m_new);
            sum = warp_sum(sum);
            if (lane == 0) {
              sl[e] = (m_old == -INFINITY ? 0.f : sl[e] * expf(m_old - m_new)) + sum;
              sm[e] = m_new;
            }
          }
          continue;
        }
        for (int e = threadIdx.x; e < nq * H * KT; e += kMixThreads) {
          const float sc = sS[e];
          sS[e] = sc == -INFINITY ? 0.f : expf(sc - sm[e / KT]) / sl[e / KT];
        }
        __syncthreads();
        for (int e = threadIdx.x; e < nq * H * KT; e += kMixThreads) {   // mixture across heads
          const int j = e % KT, h = (e / KT) % H, qi = e / (KT * H);
          const float* w = sS + qi * H * KT + j;
          float m = 0.f;
          for (int g = 0; g < H; ++g) m = fmaf(sT[h * H + g], w[g * KT], m);
          sP[e] = m;
        }
        __syncthreads();
#pragma unroll
        for (int n = 0; n < NI; ++n) {                             // weighted values: 16 bytes of one head's channels per thread
          const int e = threadIdx.x + n * kMixThreads;
          if (e < n_out) {
            const int h = e / dvc, c = e % dvc;
            const T* vv = vc + (h / rep) * dv + c * VW;
            const float* pw = sP + h * KT;
#pragma unroll 4
            for (int j = 0; j < nk; ++j) {
              float val[VW];
              Vec16<T>::load(vv + static_cast<int64_t>(sslot[j]) * G * dv, val);
#pragma unroll
              for (int qi = 0; qi < QB; ++qi) {
                const float w = pw[qi * H * KT + j];
#pragma unroll
                for (int u = 0; u < VW; ++u) acc[n][qi][u] = fmaf(w, val[u], acc[n][qi][u]);
              }
            }
          }
        }
      }
    }
    if (MODE == 1) {
      __syncthreads();
      for (int e = threadIdx.x; e < nq * H; e += kMixThreads) {
        float* ws = p.ws_stats + ((static_cast<int64_t>(seg_lo + e / H) * p.n_splits + z) * H + e % H) * 2;
        ws[0] = sm[e]; ws[1] = sl[e];
      }
    } else {
#pragma unroll
      for (int n = 0; n < NI; ++n) {
        const int e = threadIdx.x + n * kMixThreads;
        if (e >= n_out) continue;
#pragma unroll
        for (int qi = 0; qi < QB; ++qi) {
          if (qi >= nq) continue;
          const int64_t t = seg_lo + qi;
          if (MODE == 2) {
            float* dst = p.ws_acc + (t * p.n_splits + z) * H * dv + e * VW;
#pragma unroll
            for (int u = 0; u < VW; ++u) dst[u] = acc[n][qi][u];
          } else {
            float o[VW];
#pragma unroll
            for (int u = 0; u < VW; ++u) o[u] = acc[n][qi][u];
            if (p.gate != nullptr) {
              float gv[VW];
              Vec16<T>::load(static_cast<const T*>(p.gate) + t * p.ldg + e * VW, gv);
#pragma unroll
              for (int u = 0; u < VW; ++u) o[u] *= sigmoidf_(gv[u]);
            }
            Vec16<T>::store(static_cast<T*>(p.out) + t * H * dv + e * VW, o);
          }
        }
      }
    }
    seg_lo = seg_hi;
  }
}

template <typename T>
__global__ void mixed_attention_merge_kernel(MixAttnArgs p, int n_tok) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int n = p.H * p.dv;
  if (idx >= static_cast<int64_t>(n_tok) * n) return;
  const int64_t t = idx / n;
  const int e = static_cast<int>(idx % n);
  float v = 0.f;
  for (int z = 0; z < p.n_splits; ++z) v += p.ws_acc[(t * p.n_splits + z) * n + e];
  if (p.gate != nullptr) v *= sigmoidf_(ld(static_cast<const T*>(p.gate) + t * p.ldg + e));
  st(static_cast<T*>(p.out) + idx, v);
}

// ---------------------------------------------------------------------------------------------------------------------
// Generalized delta rule.  Per head, per token, with the unit key u = k / sqrt(sum k^2 + unit_eps):
//   S <- diag(w) S - (a * u) (u^T S) + k v^T   (decay and removal both act on the previous S);   o = S^T r
//   w = exp(-decay_scale * sigmoid(w_pre + w_bias)),  a = sigmoid(a_pre)
// Layout as the gated delta-rule scan of seqmix.cu: grid (column blocks, heads, sequences), a column of S shared by kParts
// lanes, a chunk of tokens staged in shared memory (decays, removal rates and unit keys are made there, in fp32).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kParts = 4;
constexpr int kScanThreads = 128;
constexpr int kColsPerCta = kScanThreads / kParts;
template <int D> struct GenChunk { static constexpr int value = D > 128 ? 4 : (D > 64 ? 8 : 16); };   // tokens staged in shared memory at a time

__device__ __forceinline__ float part_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

template <typename T, int D, bool LONG>
__global__ void __launch_bounds__(kScanThreads) gen_delta_scan_kernel(GenDeltaArgs p) {
  constexpr int CH = GenChunk<D>::value, RP = D / kParts;
  // per (token, key channel): x = unit key u, y = a * u, z = decay w, w = key k; the receptance r apart
  __shared__ float4 sx[CH][D];
  __shared__ float sr[CH][D];
  __shared__ float sv[CH][kColsPerCta];
  const int h = blockIdx.y, r = blockIdx.z;
  const int part = threadIdx.x & (kParts - 1);
  const int col = blockIdx.x * kColsPerCta + (threadIdx.x >> 2);
  const bool live = col < p.dv;
  const int a = p.cu[r], b = p.cu[r + 1];
  if (a >= b) return;
  float* state = p.state + (static_cast<int64_t>(p.rows[r]) * p.H + h) * p.d * p.dv;
  float S[RP];
#pragma unroll
  for (int e = 0; e < RP; ++e) {
    const int i = e * kParts + part;
    S[e] = (live && i < p.d) ? state[static_cast<int64_t>(i) * p.dv + col] : 0.f;
  }
  const T* rr = static_cast<const T*>(p.r);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const T* wpre = static_cast<const T*>(p.w_pre);
  const T* apre = static_cast<const T*>(p.a_pre);
  const T* wb = static_cast<const T*>(p.w_bias);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = kScanThreads >> 5;
  // The next chunk's inputs are fetched into registers before the sequential part of the current one, so that their latency
  // hides behind it; they move to shared memory (decay and removal rate made on the way) once the current chunk is done.
  // (The widest instance has no registers to spare for that and fetches in place.)
  constexpr bool PF = LONG && D <= 128;          // decoding keeps the registers for occupancy
  constexpr int NS = PF ? CH * D / kScanThreads : 1, NV = PF ? (CH * kColsPerCta + kScanThreads - 1) / kScanThreads : 1;
  float pr[NS], pk[NS], pw[NS], pa[NS], pv[NV];
  auto prefetch = [&](int t0, int nt) {
    if constexpr (!PF) return;
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int e = threadIdx.x + s * kScanThreads, tt = e / D, i = e % D;
      const int64_t t = t0 + tt;
      const bool in = tt < nt && i < p.d;
      const int c = h * p.d + i;
      pr[s] = in ? ld(rr + t * p.ldr + c) : 0.f;
      pk[s] = in ? ld(k + t * p.ldk + c) : 0.f;
      pw[s] = in ? ld(wpre + t * p.ldw + c) + (wb != nullptr ? ld(wb + c) : 0.f) : -INFINITY;   // sigmoid(-inf) = 0: decay 1
      pa[s] = in ? ld(apre + t * p.lda + c) : -INFINITY;
    }
#pragma unroll
    for (int s = 0; s < NV; ++s) {
      const int e = threadIdx.x + s * kScanThreads, tt = e / kColsPerCta, c = blockIdx.x * kColsPerCta + e % kColsPerCta;
      pv[s] = (tt < nt && c < p.dv) ? ld(v + static_cast<int64_t>(t0 + tt) * p.ldv + h * p.dv + c) : 0.f;
    }
  };
  prefetch(a, min(CH, b - a));
  for (int t0 = a; t0 < b; t0 += CH) {
    const int nt = min(CH, b - t0);
    __syncthreads();                                  // the previous chunk has been consumed
    if constexpr (PF) {
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const int e = threadIdx.x + s * kScanThreads, tt = e / D, i = e % D;
        if (tt < nt) {
          sx[tt][i] = make_float4(0.f, sigmoidf_(pa[s]), expf(-p.decay_scale * sigmoidf_(pw[s])), pk[s]);
          sr[tt][i] = pr[s];
        }
      }
#pragma unroll
      for (int s = 0; s < NV; ++s) {
        const int e = threadIdx.x + s * kScanThreads;
        if (e < nt * kColsPerCta) sv[e / kColsPerCta][e % kColsPerCta] = pv[s];
      }
    } else {
      for (int e = threadIdx.x; e < nt * D; e += kScanThreads) {
        const int tt = e / D, i = e % D, c = h * p.d + i;
        const int64_t t = t0 + tt;
        const bool in = i < p.d;
        const float wz = in ? ld(wpre + t * p.ldw + c) + (wb != nullptr ? ld(wb + c) : 0.f) : -INFINITY;
        sx[tt][i] = make_float4(0.f, in ? sigmoidf_(ld(apre + t * p.lda + c)) : 0.f, expf(-p.decay_scale * sigmoidf_(wz)),
                                in ? ld(k + t * p.ldk + c) : 0.f);
        sr[tt][i] = in ? ld(rr + t * p.ldr + c) : 0.f;
      }
      for (int e = threadIdx.x; e < nt * kColsPerCta; e += kScanThreads) {
        const int tt = e / kColsPerCta, c = blockIdx.x * kColsPerCta + e % kColsPerCta;
        sv[tt][e % kColsPerCta] = c < p.dv ? ld(v + static_cast<int64_t>(t0 + tt) * p.ldv + h * p.dv + c) : 0.f;
      }
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += n_warps) {     // unit keys and the removal direction a * u
      float kk = 0.f;
      for (int i = lane; i < D; i += 32) kk += sx[tt][i].w * sx[tt][i].w;
      kk = warp_sum(kk);
      const float rk = 1.0f / sqrtf(kk + p.unit_eps);
      for (int i = lane; i < D; i += 32) {
        const float u = sx[tt][i].w * rk;
        sx[tt][i].x = u;
        sx[tt][i].y *= u;
      }
    }
    __syncthreads();
    if (t0 + CH < b) prefetch(t0 + CH, min(CH, b - t0 - CH));
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      const float vv = sv[tt][threadIdx.x >> 2];
      constexpr bool KEEP = RP <= 16;                 // small key dims keep the token's operands in registers between the two loops
      float4 x[KEEP ? RP : 1];
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int e = 0; e < RP; e += 2) {
        if constexpr (KEEP) {
          x[e] = sx[tt][e * kParts + part];
          x[e + 1] = sx[tt][(e + 1) * kParts + part];
          d0 = fmaf(S[e], x[e].x, d0);
          d1 = fmaf(S[e + 1], x[e + 1].x, d1);
        } else {
          d0 = fmaf(S[e], sx[tt][e * kParts + part].x, d0);
          d1 = fmaf(S[e + 1], sx[tt][(e + 1) * kParts + part].x, d1);
        }
      }
      const float dot = part_sum(d0 + d1);
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int e = 0; e < RP; e += 2) {
        float4 xa, xb;
        if constexpr (KEEP) { xa = x[e]; xb = x[e + 1]; }
        else { xa = sx[tt][e * kParts + part]; xb = sx[tt][(e + 1) * kParts + part]; }
        S[e] = fmaf(xa.z, S[e], fmaf(-xa.y, dot, xa.w * vv));
        o0 = fmaf(S[e], sr[tt][e * kParts + part], o0);
        S[e + 1] = fmaf(xb.z, S[e + 1], fmaf(-xb.y, dot, xb.w * vv));
        o1 = fmaf(S[e + 1], sr[tt][(e + 1) * kParts + part], o1);
      }
      const float o = part_sum(o0 + o1);
      if (live && part == 0) p.out[(static_cast<int64_t>(t0 + tt) * p.H + h) * p.dv + col] = o;
    }
  }
  if (live) {
#pragma unroll
    for (int e = 0; e < RP; ++e) {
      const int i = e * kParts + part;
      if (i < p.d) state[static_cast<int64_t>(i) * p.dv + col] = S[e];
    }
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// minGRU: per channel  z = sigmoid(z_pre),  c = u + 1/2 (u >= 0) or sigmoid(u) (u < 0),  S <- (1 - z) S + z c,
// y = S * silu(g).  A sequence is cut into runs of kGruRun tokens.  Short sequences: one kernel walks a run from the carried state.
// Long sequences: every run first reduces to (P, Q) with S_end = P S_begin + Q, a second kernel walks the runs of a sequence to
// find each run's S_begin (and the final state), a third walks every run again from its S_begin and writes y.
// grid (channel blocks, runs, sequences); a thread owns one channel.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kGruRun = 64;
constexpr int kGruThreads = 128;
constexpr int kGruBatch = 8;

__device__ __forceinline__ void gru_gates(float zp, float up, float* z, float* c) {
  *z = sigmoidf_(zp);
  *c = up >= 0.f ? up + 0.5f : sigmoidf_(up);
}

template <typename T>
__global__ void __launch_bounds__(kGruThreads) mingru_reduce_kernel(MinGruArgs p) {
  const int c = blockIdx.x * kGruThreads + threadIdx.x, r = blockIdx.z;
  const int a = p.cu[r] + blockIdx.y * kGruRun, b = min(p.cu[r + 1], a + kGruRun);
  if (c >= p.C || a >= b) return;
  const T* zp = static_cast<const T*>(p.z_pre);
  const T* up = static_cast<const T*>(p.u_pre);
  float P = 1.f, Q = 0.f;
  for (int64_t t0 = a; t0 < b; t0 += kGruBatch) {     // the loads of a batch of tokens are issued before the dependent chain
    float zv[kGruBatch], uv[kGruBatch];
#pragma unroll
    for (int j = 0; j < kGruBatch; ++j) {
      const bool in = t0 + j < b;
      zv[j] = in ? ld(zp + (t0 + j) * p.ldz + c) : 0.f;
      uv[j] = in ? ld(up + (t0 + j) * p.ldu + c) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kGruBatch; ++j) {
      if (t0 + j < b) {
        float z, cand;
        gru_gates(zv[j], uv[j], &z, &cand);
        P *= 1.f - z;
        Q = fmaf(1.f - z, Q, z * cand);
      }
    }
  }
  float* ws = p.ws + ((static_cast<int64_t>(r) * p.max_runs + blockIdx.y) * p.C + c) * 2;
  ws[0] = P; ws[1] = Q;
}

__global__ void __launch_bounds__(kGruThreads) mingru_carry_kernel(MinGruArgs p) {
  const int c = blockIdx.x * kGruThreads + threadIdx.x, r = blockIdx.z;
  const int n = p.cu[r + 1] - p.cu[r];
  if (c >= p.C || n <= 0) return;
  float* st_ = p.state + static_cast<int64_t>(p.rows[r]) * p.C + c;
  float S = *st_;
  const int runs = (n + kGruRun - 1) / kGruRun;
  for (int y = 0; y < runs; ++y) {
    float* ws = p.ws + ((static_cast<int64_t>(r) * p.max_runs + y) * p.C + c) * 2;
    const float P = ws[0], Q = ws[1];
    ws[0] = S;                                        // the run's starting state, for the third kernel
    S = fmaf(P, S, Q);
  }
  *st_ = S;
}

template <typename T, bool CARRIED>
__global__ void __launch_bounds__(kGruThreads) mingru_apply_kernel(MinGruArgs p) {
  const int c = blockIdx.x * kGruThreads + threadIdx.x, r = blockIdx.z;
  const int a0 = p.cu[r], b0 = p.cu[r + 1];
  const int a = CARRIED ? a0 + blockIdx.y * kGruRun : a0, b = CARRIED ? min(b0, a + kGruRun) : b0;
  if (c >= p.C || a >= b) return;
  const T* zp = static_cast<const T*>(p.z_pre);
  const T* up = static_cast<const T*>(p.u_pre);
  const T* gp = static_cast<const T*>(p.g_pre);
  T* y = static_cast<T*>(p.y);
  float* st_ = p.state + static_cast<int64_t>(p.rows[r]) * p.C + c;
  float S = CARRIED ? p.ws[((static_cast<int64_t>(r) * p.max_runs + blockIdx.y) * p.C + c) * 2] : *st_;
  for (int64_t t0 = a; t0 < b; t0 += kGruBatch) {
    float zv[kGruBatch], uv[kGruBatch], gv[kGruBatch];
#pragma unroll
    for (int j = 0; j < kGruBatch; ++j) {
      const bool in = t0 + j < b;
      zv[j] = in ? ld(zp + (t0 + j) * p.ldz + c) : 0.f;
      uv[j] = in ? ld(up + (t0 + j) * p.ldu + c) : 0.f;
      gv[j] = in ? ld(gp + (t0 + j) * p.ldg + c) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < kGruBatch; ++j) {
      if (t0 + j < b) {
        float z, cand;
        gru_gates(zv[j], uv[j], &z, &cand);
        S = fmaf(1.f - z, S, z * cand);
        st(y + (t0 + j) * p.C + c, S * gv[j] * sigmoidf_(gv[j]));
      }
    }
  }
  if (!CARRIED) *st_ = S;
}

// ---------------------------------------------------------------------------------------------------------------------
// clamped gated activation over [gate | up] rows: g = min(gate, limit), u = clamp(up, -limit, limit),
// y = g * sigmoid(alpha * g) * (u + shift)
// ---------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void clamped_glu_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y, int64_t n_tok, int F, float limit,
                                   float alpha, float shift) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n_tok * F) return;
  const int64_t t = idx / F;
  const int c = static_cast<int>(idx % F);
  const float g = fminf(ld(x + t * ldx + c), limit);
  const float u = fminf(fmaxf(ld(x + t * ldx + F + c), -limit), limit);
  st(y + idx, g * sigmoidf_(alpha * g) * (u + shift));
}

template <typename T>
__global__ void clamped_glu_vec_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y, int64_t n_tok, int F, float limit,
                                       float alpha, float shift) {
  constexpr int VW = Vec16<T>::W;
  const int per_row = F / VW;
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n_tok * per_row) return;
  const int64_t t = idx / per_row;
  const int c = static_cast<int>(idx % per_row) * VW;
  float g[VW], u[VW], o[VW];
  Vec16<T>::load(x + t * ldx + c, g);
  Vec16<T>::load(x + t * ldx + F + c, u);
#pragma unroll
  for (int i = 0; i < VW; ++i) {
    const float gg = fminf(g[i], limit), uu = fminf(fmaxf(u[i], -limit), limit);
    o[i] = gg * sigmoidf_(alpha * gg) * (uu + shift);
  }
  Vec16<T>::store(y + t * F + c, o);
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------------
void norm_add(float* x, const void* a, const void* b, const void* wa, const void* wb, const void* w, void* y, int rows, int cols,
              float eps, float w_off, const void* extra, const void* next_w, bool bf16, cudaStream_t s) {
  if (rows == 0) return;
  SEQ_DISPATCH_T(bf16, norm_add_kernel<T><<<rows, 256, cols * sizeof(float), s>>>(
                           x, static_cast<const T*>(a), static_cast<const T*>(b), static_cast<const T*>(wa),
                           static_cast<const T*>(wb), static_cast<const T*>(w), static_cast<T*>(y), cols, eps, w_off,
                           static_cast<const T*>(extra), static_cast<const T*>(next_w)));
}

void norm_rope(const NormRopeArgs& p, int n_tok, bool bf16, cudaStream_t s) {
  if (n_tok == 0) return;
  const size_t smem = static_cast<size_t>(std::max(p.q_ch, p.k_ch) + 1 + p.rot) * sizeof(float);
  const size_t two = bf16 ? 4 : 8;
  auto al = [&](const void* q) { return reinterpret_cast<uintptr_t>(q) % two == 0; };
  const bool paired = p.head_dim % 2 == 0 && p.ldq % 2 == 0 && p.ldk % 2 == 0 && al(p.q) && al(p.k) && al(p.wq) && al(p.wk) &&
                      al(p.q_out) && al(p.k_out);
  SEQ_DISPATCH_T(bf16, {
    if (paired) norm_rope_kernel<T, true><<<dim3(n_tok, 2), 256, smem, s>>>(p);
    else norm_rope_kernel<T, false><<<dim3(n_tok, 2), 256, smem, s>>>(p);
  });
}

int mixed_attention_splits(int n_tok, int max_len) {
  if (n_tok >= 2 * 148 || max_len < 1024) return 1;
  const int want = (4 * 148 + n_tok - 1) / n_tok;
  return std::max(1, std::min(std::min(want, 32), max_len / 256));
}

// shared-memory plan: words of the fp32 / int part (a multiple of 4), the padded key row, and the key tile that fits
static size_t mix_smem(const MixAttnArgs& p, int kt, size_t elt, int* head_words, int* ldk) {
  int words = p.H * p.d + 2 * p.H * kt + p.H * p.H + 2 * p.H + kt;
  words = (words + 3) / 4 * 4;
  const int row = p.G * p.d;
  int pad = row;
  if (elt == 4) { if (pad % 2 == 0) pad += 1; }                    // an odd number of 32-bit words per key row
  else { if (pad % 2) pad += 1; if ((pad / 2) % 2 == 0) pad += 2; }
  *head_words = words; *ldk = pad;
  return static_cast<size_t>(words) * 4 + static_cast<size_t>(kt) * (pad + p.G * p.dv) * elt;
}

template <typename T, int NACC>
static bool launch_mix(MixAttnArgs p, int n_tok, cudaStream_t s) {
  int kt = 128;
  size_t smem = 0;
  for (; kt >= 8; kt /= 2) {
    smem = mix_smem(p, kt, sizeof(T), &p.head_words, &p.ldk_s);
    if (smem <= 100 * 1024) break;
  }
  if (kt < 8) return false;
  p.key_tile = kt;
  auto set = [&](auto kern) {
    return smem <= 48 * 1024 || cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess;
  };
  if (p.n_splits == 1) {
    auto kern = mixed_attention_kernel<T, NACC, 0>;
    if (!set(kern)) return false;
    kern<<<dim3(n_tok, 1), kMixThreads, smem, s>>>(p);
    return true;
  }
  auto k1 = mixed_attention_kernel<T, NACC, 1>;
  auto k2 = mixed_attention_kernel<T, NACC, 2>;
  if (!set(k1) || !set(k2)) return false;
  k1<<<dim3(n_tok, p.n_splits), kMixThreads, smem, s>>>(p);
  k2<<<dim3(n_tok, p.n_splits), kMixThreads, smem, s>>>(p);
  const int64_t n = static_cast<int64_t>(n_tok) * p.H * p.dv;
  mixed_attention_merge_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(p, n_tok);
  return true;
}

// the vector kernel's shared-memory plan for a query block of qb tokens and a tile of kt keys
static size_t vec_smem(const MixAttnArgs& p, int qb, int kt, size_t elt, int* head_words, int* ldk) {
  int words = qb * p.H * p.d + 2 * qb * p.H * kt + p.H * p.H + 2 * qb * p.H + kt + qb;
  words = (words + 3) / 4 * 4;
  const size_t row_bytes = (static_cast<size_t>(p.G) * p.d * elt + 127) / 128 * 128 + 16;
  *head_words = words; *ldk = static_cast<int>(row_bytes / elt);
  return static_cast<size_t>(words) * 4 + static_cast<size_t>(kt) * row_bytes;
}

template <typename T, int NI, int QB>
static bool launch_vec(MixAttnArgs p, int n_tok, int kt, cudaStream_t s) {
  const size_t smem = vec_smem(p, QB, kt, sizeof(T), &p.head_words, &p.ldk_s);
  p.key_tile = kt;
  auto set = [&](auto kern) {
    return smem <= 48 * 1024 || cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) == cudaSuccess;
  };
  const int blocks = (n_tok + QB - 1) / QB;
  if (p.n_splits == 1) {
    auto kern = mixed_attention_vec_kernel<T, NI, QB, 0>;
    if (!set(kern)) return false;
    kern<<<dim3(blocks, 1), kMixThreads, smem, s>>>(p, n_tok);
    return true;
  }
  auto k1 = mixed_attention_vec_kernel<T, NI, QB, 1>;
  auto k2 = mixed_attention_vec_kernel<T, NI, QB, 2>;
  if (!set(k1) || !set(k2)) return false;
  k1<<<dim3(blocks, p.n_splits), kMixThreads, smem, s>>>(p, n_tok);
  k2<<<dim3(blocks, p.n_splits), kMixThreads, smem, s>>>(p, n_tok);
  const int64_t n = static_cast<int64_t>(n_tok) * p.H * p.dv;
  mixed_attention_merge_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(p, n_tok);
  return true;
}

// 0: sizes or alignment the vector kernel does not take; 1: launched; -1: launch failed
template <typename T>
static int try_vec(const MixAttnArgs& p, int n_tok, cudaStream_t s) {
  constexpr int VW = Vec16<T>::W;
  auto al = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  if (p.d % VW || p.dv % VW || p.ldq % VW || !al(p.q) || !al(p.kcache) || !al(p.vcache) || !al(p.out) ||
      (p.gate != nullptr && (!al(p.gate) || p.ldg % VW)))
    return 0;
  const int ni = (p.H * p.dv / VW + kMixThreads - 1) / kMixThreads;
  if (ni > 4) return 0;
  // several queries per CTA once the step brings many tokens per sequence and the grid still fills the GPU
  int qb = (p.query_block >= 4 && p.n_splits == 1 && ni <= 2) ? 4 : 1;
  int hw, ldk, kt = 0;
  for (;; qb = 1) {
    for (kt = 64; kt >= 16; kt /= 2)
      if (vec_smem(p, qb, kt, sizeof(T), &hw, &ldk) <= 96 * 1024) break;
    if (kt >= 16 || qb == 1) break;
  }
  if (kt < 16) return 0;
  bool ok = false;
  if (qb == 4) ok = ni == 1 ? launch_vec<T, 1, 4>(p, n_tok, kt, s) : launch_vec<T, 2, 4>(p, n_tok, kt, s);
  else if (ni == 1) ok = launch_vec<T, 1, 1>(p, n_tok, kt, s);
  else if (ni == 2) ok = launch_vec<T, 2, 1>(p, n_tok, kt, s);
  else ok = launch_vec<T, 4, 1>(p, n_tok, kt, s);
  return ok ? 1 : -1;
}

template <typename T>
static bool dispatch_mix(const MixAttnArgs& p, int n_tok, cudaStream_t s) {
  if (!p.force_generic) {
    const int v = try_vec<T>(p, n_tok, s);
    if (v != 0) return v > 0;
  }
  const int per = (p.H * p.dv + kMixThreads - 1) / kMixThreads;
  if (per <= 1) return launch_mix<T, 1>(p, n_tok, s);
  if (per <= 2) return launch_mix<T, 2>(p, n_tok, s);
  if (per <= 4) return launch_mix<T, 4>(p, n_tok, s);
  if (per <= 8) return launch_mix<T, 8>(p, n_tok, s);
  if (per <= 16) return launch_mix<T, 16>(p, n_tok, s);
  if (per <= 32) return launch_mix<T, 32>(p, n_tok, s);
  return false;
}

bool mixed_attention_paged(const MixAttnArgs& p, int n_tok, bool bf16, cudaStream_t s) {
  if (n_tok == 0) return true;
  if (p.H % p.G != 0) return false;
  return bf16 ? dispatch_mix<__nv_bfloat16>(p, n_tok, s) : dispatch_mix<float>(p, n_tok, s);
}

template <typename T>
static bool launch_gen_delta(const GenDeltaArgs& p, dim3 grid, cudaStream_t s) {
#define SEQ_GEN_DELTA(DD)                                                                                       \
  if (p.max_len > GenChunk<DD>::value) gen_delta_scan_kernel<T, DD, true><<<grid, kScanThreads, 0, s>>>(p);     \
  else gen_delta_scan_kernel<T, DD, false><<<grid, kScanThreads, 0, s>>>(p)
  if (p.d <= 32) { SEQ_GEN_DELTA(32); }
  else if (p.d <= 64) { SEQ_GEN_DELTA(64); }
  else if (p.d <= 128) { SEQ_GEN_DELTA(128); }
  else if (p.d <= 256) { SEQ_GEN_DELTA(256); }
  else return false;
#undef SEQ_GEN_DELTA
  return true;
}

bool gen_delta_scan(const GenDeltaArgs& p, int R, bool bf16, cudaStream_t s) {
  if (R == 0) return true;
  dim3 grid((p.dv + kColsPerCta - 1) / kColsPerCta, p.H, R);
  return bf16 ? launch_gen_delta<__nv_bfloat16>(p, grid, s) : launch_gen_delta<float>(p, grid, s);
}

int mingru_runs(int max_len) { return max_len > 4 * kGruRun ? (max_len + kGruRun - 1) / kGruRun : 1; }

void mingru_scan(const MinGruArgs& p, int R, bool bf16, cudaStream_t s) {
  if (R == 0 || p.C == 0) return;
  const int cb = (p.C + kGruThreads - 1) / kGruThreads;
  if (p.max_runs <= 1) {
    SEQ_DISPATCH_T(bf16, mingru_apply_kernel<T, false><<<dim3(cb, 1, R), kGruThreads, 0, s>>>(p));
    return;
  }
  SEQ_DISPATCH_T(bf16, mingru_reduce_kernel<T><<<dim3(cb, p.max_runs, R), kGruThreads, 0, s>>>(p));
  mingru_carry_kernel<<<dim3(cb, 1, R), kGruThreads, 0, s>>>(p);
  SEQ_DISPATCH_T(bf16, mingru_apply_kernel<T, true><<<dim3(cb, p.max_runs, R), kGruThreads, 0, s>>>(p));
}

void clamped_glu(const void* x, int64_t ldx, void* y, int64_t n_tok, int F, float limit, float alpha, float shift, bool bf16,
                 cudaStream_t s) {
  const int64_t n = n_tok * F;
  if (n == 0) return;
  const int vw = bf16 ? 8 : 4;
  if (F % vw == 0 && ldx % vw == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0) {
    const int64_t nv = n / vw;
    SEQ_DISPATCH_T(bf16, clamped_glu_vec_kernel<T><<<static_cast<unsigned>((nv + 255) / 256), 256, 0, s>>>(
                             static_cast<const T*>(x), ldx, static_cast<T*>(y), n_tok, F, limit, alpha, shift));
    return;
  }
  SEQ_DISPATCH_T(bf16, clamped_glu_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(
                           static_cast<const T*>(x), ldx, static_cast<T*>(y), n_tok, F, limit, alpha, shift));
}

}  // namespace b200seq
