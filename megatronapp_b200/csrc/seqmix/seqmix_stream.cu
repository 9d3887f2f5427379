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
constexpr int kMaxStreams = 8;

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
// all keys up to i); score = q . k * scale - slope[h] * (i - j); weights exp(s_j) / (sink + sum_j exp(s_j)) where the sink
// (0 or 1) is a key of score 0 without a value; the head's output is multiplied by sigmoid(gate[t, h]) and out_scale.
//
// grid (query blocks, kv heads, head chunks).  A CTA takes QB consecutive packed tokens and HC heads of one kv head: its
// QB * HC <= 32 (query, head) pairs are spread over 8 warps, 4 pairs each.  Keys and values of a tile of 32 cached tokens are
// staged in shared memory as fp32 once for all pairs.  Scores: a lane owns one key of the tile and walks the head dimension
// for the warp's 4 pairs at once; the online softmax state (m, l) is kept per pair; values: a lane owns channels
// lane, lane + 32, ... of the 4 accumulators.  A block of tokens that straddles sequences walks them one after the other.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kWinWarps = 8, kWinPairs = 4, kWinTile = 32;

template <typename T, int DVR>
__global__ void __launch_bounds__(kWinWarps * 32) window_attention_kernel(WindowAttnArgs p) {
  extern __shared__ float smem[];
  const int d = p.d, dv = p.dv, ldk = d + 1, ldv = dv;
  float* sq = smem;                                        // [32 pairs][d]
  float* sk = sq + 32 * d;                                 // [tile][d + 1]
  float* sv = sk + kWinTile * ldk;                         // [tile][dv]
  float* sp = sv + kWinTile * ldv;                         // [warps][pairs][tile]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = blockIdx.y, rep = p.H / p.G;
  const int h_lo = blockIdx.z * p.HC, n_heads = min(p.HC, rep - h_lo);     // heads of this chunk, relative to the group
  const int t0 = blockIdx.x * p.QB, t1 = min(p.n_tok, t0 + p.QB);
  const T* qbase = static_cast<const T*>(p.q);
  const T* kc = static_cast<const T*>(p.kcache);
  const T* vc = static_cast<const T*>(p.vcache);
  float* mysp = sp + warp * kWinPairs * kWinTile;

  int seg = t0;
  while (seg < t1) {
    const int r = p.tok_req[seg];
    int seg_end = seg + 1;
    while (seg_end < t1 && p.tok_req[seg_end] == r) ++seg_end;
    const int nq = seg_end - seg, n_pairs = nq * n_heads;
    const int* table = p.block_table + static_cast<int64_t>(r) * p.max_blocks;
    const int len_first = p.tok_len[seg], len_last = p.tok_len[seg_end - 1];
    const int k_begin = p.window > 0 ? max(0, len_first - p.window) : 0, k_end = len_last;
    __syncthreads();                                       // the previous segment's reads of sq are over
    for (int i = threadIdx.x; i < n_pairs * d; i += blockDim.x) {
      const int pr = i / d, c = i % d, qi = pr / n_heads, hh = pr % n_heads;
      sq[pr * d + c] = ld(qbase + static_cast<int64_t>(seg + qi) * p.ldq + static_cast<int64_t>(g * rep + h_lo + hh) * d + c) * p.scale;
    }
    // per-pair state of this warp
    float m[kWinPairs], l[kWinPairs], acc[kWinPairs][DVR], slope[kWinPairs];
    int pos[kWinPairs], lo[kWinPairs];
#pragma unroll
    for (int u = 0; u < kWinPairs; ++u) {
      const int pr = warp * kWinPairs + u;
      m[u] = p.sink ? 0.f : -INFINITY;
      l[u] = p.sink ? 1.f : 0.f;
#pragma unroll
      for (int k = 0; k < DVR; ++k) acc[u][k] = 0.f;
      if (pr < n_pairs) {
        const int qi = pr / n_heads, hh = pr % n_heads;
        pos[u] = p.tok_len[seg + qi] - 1;
        lo[u] = p.window > 0 ? max(0, pos[u] + 1 - p.window) : 0;
        slope[u] = p.slopes != nullptr ? p.slopes[g * rep + h_lo + hh] : 0.f;
      } else { pos[u] = -1; lo[u] = 0; slope[u] = 0.f; }
    }
    for (int k0 = k_begin; k0 < k_end; k0 += kWinTile) {
      const int n_keys = min(kWinTile, k_end - k0);
      __syncthreads();                                     // the previous tile (and sq) is settled
      for (int i = threadIdx.x; i < n_keys * d; i += blockDim.x) {
        const int j = i / d, c = i % d, key = k0 + j;
        const int64_t slot = static_cast<int64_t>(table[key / p.block_size]) * p.block_size + key % p.block_size;
        sk[j * ldk + c] = ld(kc + (slot * p.G + g) * d + c);
      }
      for (int i = threadIdx.x; i < n_keys * dv; i += blockDim.x) {
        const int j = i / dv, c = i % dv, key = k0 + j;
        const int64_t slot = static_cast<int64_t>(table[key / p.block_size]) * p.block_size + key % p.block_size;
        sv[j * ldv + c] = ld(vc + (slot * p.G + g) * dv + c);
      }
      __syncthreads();
      // does any pair of this warp see a key of this tile?
      bool any = false;
#pragma unroll
      for (int u = 0; u < kWinPairs; ++u) any = any || (pos[u] >= k0 && lo[u] < k0 + n_keys);
      if (!any) continue;
      float s[kWinPairs];
#pragma unroll
      for (int u = 0; u < kWinPairs; ++u) s[u] = 0.f;
      if (lane < n_keys) {
        const float* krow = sk + lane * ldk;
        const float* q0 = sq + (warp * kWinPairs) * d;
        for (int c = 0; c < d; ++c) {
          const float kv = krow[c];
#pragma unroll
          for (int u = 0; u < kWinPairs; ++u) s[u] = fmaf(q0[u * d + c], kv, s[u]);
        }
      }
      const int key = k0 + lane;
#pragma unroll
      for (int u = 0; u < kWinPairs; ++u) {
        const bool vis = lane < n_keys && key <= pos[u] && key >= lo[u];
        const float sc = vis ? s[u] - slope[u] * static_cast<float>(pos[u] - key) : -INFINITY;
        const float m_new = fmaxf(m[u], warp_max(sc));
        float pw = 0.f, corr = 1.f;
        if (m_new != -INFINITY) {
          pw = vis ? expf(sc - m_new) : 0.f;
          corr = expf(m[u] - m_new);                      // m = -inf: 0, and l and acc are 0 then
        }
        l[u] = l[u] * corr + warp_sum(pw);
        m[u] = m_new;
#pragma unroll
        for (int k = 0; k < DVR; ++k) acc[u][k] *= corr;
        mysp[u * kWinTile + lane] = pw;
      }
      __syncwarp();
      for (int j = 0; j < n_keys; ++j) {
        float pj[kWinPairs];
#pragma unroll
        for (int u = 0; u < kWinPairs; ++u) pj[u] = mysp[u * kWinTile + j];
#pragma unroll
        for (int k = 0; k < DVR; ++k) {
          const int c = lane + 32 * k;
          if (c < dv) {
            const float vv = sv[j * ldv + c];
#pragma unroll
            for (int u = 0; u < kWinPairs; ++u) acc[u][k] = fmaf(pj[u], vv, acc[u][k]);
          }
        }
      }
      __syncwarp();
    }
    // write the pairs of this warp
    T* out = static_cast<T*>(p.out);
    const T* gate = static_cast<const T*>(p.gate);
#pragma unroll
    for (int u = 0; u < kWinPairs; ++u) {
      const int pr = warp * kWinPairs + u;
      if (pr >= n_pairs) continue;
      const int qi = pr / n_heads, hh = pr % n_heads, head = g * rep + h_lo + hh;
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
  float* sB = sx + kSelChunk * kSelCh;               // [chunk][N]
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
    A[i] = ok ? -expf(ld(static_cast<const T*>(p.A_log) + static_cast<int64_t>(c) * N + n)) : 0.f;
    S[i] = ok ? st_row[n] : 0.f;
  }
  const float Dc = live ? ld(static_cast<const T*>(p.D) + c) : 0.f;
  for (int t0 = a; t0 < b; t0 += kSelChunk) {
    const int nt = min(kSelChunk, b - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * kSelCh; i += kSelThreads) {
      const int tt = i / kSelCh, cc = i % kSelCh;
      float dtv = 0.f, xv = 0.f;
      if (c0 + cc < p.C) {
        const float pre = p.dt_pre[static_cast<int64_t>(t0 + tt) * p.lddt + c0 + cc] +
                          (p.dt_bias != nullptr ? ld(static_cast<const T*>(p.dt_bias) + c0 + cc) : 0.f);
        dtv = pre > 20.f ? pre : log1pf(expf(pre));
        xv = ld(x + static_cast<int64_t>(t0 + tt) * p.ldx + c0 + cc);
      }
      sdt[i] = dtv; sx[i] = xv;
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
          S[i] = fmaf(expf(dtv * A[i]), S[i], dx * sB[tt * N + n]);
          acc = fmaf(S[i], sC[tt * N + n], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (live && part == 0) {
        const int64_t t = t0 + tt;
        float v = fmaf(Dc, xv, acc);
        if (z != nullptr) { const float zv = ld(z + t * p.ldz + c); v *= zv * sigmoidf_(zv); }
        st(y + t * p.ldy + c, v * p.out_scale);
      }
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
  SEQ_DISPATCH_T(bf16, {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(stream_mix_norm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    stream_mix_norm_kernel<T><<<n_tok, 256, smem, s>>>(p);
  });
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

template <typename T, int DVR>
static bool launch_window(WindowAttnArgs& p, cudaStream_t s) {
  const int rep = p.H / p.G;
  p.HC = std::min(rep, kWinWarps * kWinPairs);
  p.QB = std::max(1, (kWinWarps * kWinPairs) / p.HC);
  const size_t smem = (static_cast<size_t>(32) * p.d + static_cast<size_t>(kWinTile) * (p.d + 1) + static_cast<size_t>(kWinTile) * p.dv +
                       static_cast<size_t>(kWinWarps) * kWinPairs * kWinTile) * sizeof(float);
  if (smem > 220 * 1024) return false;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(window_attention_kernel<T, DVR>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  dim3 grid((p.n_tok + p.QB - 1) / p.QB, p.G, (rep + p.HC - 1) / p.HC);
  window_attention_kernel<T, DVR><<<grid, kWinWarps * 32, smem, s>>>(p);
  return true;
}

bool window_attention_paged(const WindowAttnArgs& p_in, bool bf16, cudaStream_t s) {
  WindowAttnArgs p = p_in;
  if (p.n_tok == 0) return true;
  if (p.H % p.G != 0 || p.G > 65535) return false;
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
  const size_t smem = (2 * static_cast<size_t>(kSelChunk) * kSelCh + 2 * static_cast<size_t>(kSelChunk) * p.N) * sizeof(float);
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
