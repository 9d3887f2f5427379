// Sequence-mixing kernels over a packed token batch (sm_100a): fp32-residual RMS norms, short causal convolution with a
// carried window, gated delta-rule and mLSTM matrix-memory scans, latent attention over a paged cache, group-limited router.
//
// Conventions: activations are `T` (float or __nv_bfloat16); statistics, gates, decays, scores and every recurrent state are
// fp32.  `cu[R + 1]` holds the sequence boundaries of the packed batch, `rows[R]` the state row of every sequence.
// The scans keep the d x dv memory in registers, a column per group of four lanes (columns never interact), stage q / k /
// gates of a chunk of tokens in shared memory, and therefore synchronise a few times per chunk instead of per token.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <algorithm>

#include "seq_common.cuh"
#include "seqmix_api.h"

namespace b200seq {

namespace {

using namespace dev;

// ---------------------------------------------------------------------------------------------------------------------
// x (fp32, in place) += delta ; y = x * rsqrt(mean(x^2) + eps) * (w_off + w)
// ---------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) add_rms_norm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                                           const T* __restrict__ w, T* __restrict__ y, int cols, float eps, float w_off) {
  extern __shared__ float row[];
  __shared__ float red[8];
  const int64_t base = static_cast<int64_t>(blockIdx.x) * cols;
  float ss = 0.f;
  for (int c = threadIdx.x; c < cols; c += blockDim.x) {
    float v = x[base + c];
    if (delta != nullptr) {
      v += ld(delta + base + c);
      x[base + c] = v;
    }
    row[c] = v;
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
  const float r = 1.0f / sqrtf(tot / static_cast<float>(cols) + eps);
  for (int c = threadIdx.x; c < cols; c += blockDim.x) st(y + base + c, row[c] * r * (w_off + ld(w + c)));
}

// one warp per (token, head): o / rms(o) * w * act(gate), act = sigmoid or silu; w nullptr: no weight
template <typename T>
__global__ void gated_head_rms_norm_kernel(const float* __restrict__ o, const T* __restrict__ w, const T* __restrict__ gate, int64_t ldg,
                                           T* __restrict__ y, int n_rows, int H, int dv, int w_per_head, float eps, int silu) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31, h = row % H;
  const float* src = o + static_cast<int64_t>(row) * dv;
  float ss = 0.f;
  for (int c = lane; c < dv; c += 32) ss += src[c] * src[c];
  ss = warp_sum(ss);
  const float r = 1.0f / sqrtf(ss / static_cast<float>(dv) + eps);
  for (int c = lane; c < dv; c += 32) {
    float v = src[c] * r;
    if (w != nullptr) v *= ld(w + (w_per_head ? h * dv : 0) + c);
    if (gate != nullptr) {
      const float gv = ld(gate + static_cast<int64_t>(row / H) * ldg + h * dv + c);
      v *= silu ? gv * sigmoidf_(gv) : sigmoidf_(gv);
    }
    st(y + static_cast<int64_t>(row) * dv + c, v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// depth-wise causal convolution (+ SiLU when asked for); the window holds the taps - 1 inputs that preceded the step
// ---------------------------------------------------------------------------------------------------------------------
template <typename T>
__global__ void causal_conv_silu_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w, const T* __restrict__ bias,
                                        const int* __restrict__ cu,
                                        const int* __restrict__ rows, const int* __restrict__ tok_seq, const T* __restrict__ window,
                                        T* __restrict__ y, int n_tok, int C, int taps, int silu) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(n_tok) * C) return;
  const int t = static_cast<int>(idx / C), c = static_cast<int>(idx % C);
  const int r = tok_seq[t], a = cu[r];
  const T* win = window + static_cast<int64_t>(rows[r]) * (taps - 1) * C;
  float acc = bias != nullptr ? ld(bias + c) : 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = t - (taps - 1 - j);
    const float in = src >= a ? ld(x + src * ldx + c) : ld(win + static_cast<int64_t>(taps - 1 + (src - a)) * C + c);
    acc += ld(w + static_cast<int64_t>(c) * taps + j) * in;
  }
  if (silu & 1) acc *= sigmoidf_(acc);
  if (silu & 2) acc += ld(x + t * ldx + c);
  st(y + static_cast<int64_t>(t) * C + c, acc);
}

// Two adjacent channels and a run of kConvRun tokens of one sequence per thread: every input is read once and slides through
// registers.  grid (channel-pair blocks, runs of the longest sequence, sequences).
constexpr int kConvRun = 8;

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

template <typename T, int TAPS>
__global__ void __launch_bounds__(128) causal_conv_silu_run_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ w,
                                                                   const T* __restrict__ bias, const int* __restrict__ cu, const int* __restrict__ rows,
                                                                   const T* __restrict__ window, T* __restrict__ y, int C, int silu) {
  const int c = 2 * (blockIdx.x * blockDim.x + threadIdx.x), r = blockIdx.z;
  const int a = cu[r], b = cu[r + 1];
  const int t_lo = a + blockIdx.y * kConvRun, t_hi = min(b, t_lo + kConvRun);
  if (c >= C || t_lo >= t_hi) return;
  const T* win = window + static_cast<int64_t>(rows[r]) * (TAPS - 1) * C;
  float2 wt[TAPS], hist[TAPS];
  const float2 bs = bias != nullptr ? make_float2(ld(bias + c), ld(bias + c + 1)) : make_float2(0.f, 0.f);
#pragma unroll
  for (int j = 0; j < TAPS; ++j) wt[j] = make_float2(ld(w + static_cast<int64_t>(c) * TAPS + j), ld(w + static_cast<int64_t>(c + 1) * TAPS + j));
#pragma unroll
  for (int j = 0; j < TAPS - 1; ++j) {               // hist[j] = input at t_lo - (TAPS - 1) + j
    const int src = t_lo - (TAPS - 1) + j;
    hist[j] = src >= a ? Pair<T>::load(x + src * ldx + c) : Pair<T>::load(win + static_cast<int64_t>(TAPS - 1 + (src - a)) * C + c);
  }
  for (int t = t_lo; t < t_hi; ++t) {
    hist[TAPS - 1] = Pair<T>::load(x + t * ldx + c);
    float2 acc = bs;
#pragma unroll
    for (int j = 0; j < TAPS; ++j) { acc.x = fmaf(wt[j].x, hist[j].x, acc.x); acc.y = fmaf(wt[j].y, hist[j].y, acc.y); }
    if (silu & 1) acc = make_float2(acc.x * sigmoidf_(acc.x), acc.y * sigmoidf_(acc.y));
    if (silu & 2) { acc.x += hist[TAPS - 1].x; acc.y += hist[TAPS - 1].y; }
    Pair<T>::store(y + static_cast<int64_t>(t) * C + c, acc);
#pragma unroll
    for (int j = 0; j < TAPS - 1; ++j) hist[j] = hist[j + 1];
  }
}

template <typename T>
__global__ void conv_window_update_kernel(const T* __restrict__ x, int64_t ldx, const int* __restrict__ cu,
                                          const int* __restrict__ rows, T* __restrict__ window, int R, int C, int taps) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<int64_t>(R) * C) return;
  const int r = static_cast<int>(idx / C), c = static_cast<int>(idx % C);
  const int a = cu[r], b = cu[r + 1], n = b - a, keep = taps - 1;
  T* win = window + static_cast<int64_t>(rows[r]) * keep * C;
  for (int i = 0; i < keep; ++i) {                  // ascending: entry i + n is read before it can be overwritten
    const int src = b - keep + i;
    win[static_cast<int64_t>(i) * C + c] = src >= a ? x[src * ldx + c] : win[static_cast<int64_t>(i + n) * C + c];
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// gated delta rule.  grid (column blocks, heads, sequences).  A column of S is shared by kParts adjacent lanes: lane
// `part` keeps rows part, part + kParts, ... in registers, so the two reductions over the key dimension per token end in
// two shuffles and the dependent chains are a quarter as long.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kParts = 4;
constexpr int kScanThreads = 128;
constexpr int kColsPerCta = kScanThreads / kParts;
template <int D> struct ScanChunk { static constexpr int value = D > 128 ? 8 : 16; };   // tokens staged per shared-memory round

__device__ __forceinline__ float part_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  return v;
}

template <typename T, int D, bool PF>
__global__ void __launch_bounds__(kScanThreads) delta_rule_scan_kernel(DeltaArgs p) {
  constexpr int CH = ScanChunk<D>::value, RP = D / kParts;
  __shared__ float sq[CH][D], sk[CH][D], sg[CH][D];
  __shared__ float sv[CH][kColsPerCta];
  __shared__ float sbeta[CH];
  const int h = blockIdx.y, r = blockIdx.z, kh = h / (p.H / p.KH);
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
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = kScanThreads >> 5;
  // With PF (sequences longer than a chunk) the next chunk's inputs are fetched into registers before the sequential part of
  // the current one, so that their latency hides behind it; they move to shared memory (decays exponentiated) once the current
  // chunk is done.  Without PF (decoding) a chunk is fetched when its turn comes, which keeps the registers free for occupancy.
  constexpr int NS = CH * D / kScanThreads, NV = (CH * kColsPerCta + kScanThreads - 1) / kScanThreads;
  float pq[NS], pk[NS], pg[NS], pv[NV], pbeta = 0.f;
  auto prefetch = [&](int t0, int nt) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int e = threadIdx.x + s * kScanThreads, tt = e / D, i = e % D, t = t0 + tt;
      const bool in = tt < nt && i < p.d;
      pq[s] = in ? ld(q + t * p.ldq + kh * p.d + i) : 0.f;
      pk[s] = in ? ld(k + t * p.ldk + kh * p.d + i) : 0.f;
      pg[s] = in ? (p.decay_per_head ? p.log_decay[static_cast<int64_t>(t) * p.H + h] : p.log_decay[(static_cast<int64_t>(t) * p.H + h) * p.d + i]) : 0.f;
    }
#pragma unroll
    for (int s = 0; s < NV; ++s) {
      const int e = threadIdx.x + s * kScanThreads, tt = e / kColsPerCta, c = blockIdx.x * kColsPerCta + e % kColsPerCta;
      pv[s] = (tt < nt && c < p.dv) ? ld(v + (t0 + tt) * p.ldv + h * p.dv + c) : 0.f;
    }
    if (threadIdx.x < nt) pbeta = p.beta[static_cast<int64_t>(t0 + threadIdx.x) * p.H + h];
  };
  if (PF) prefetch(a, min(CH, b - a));
  for (int t0 = a; t0 < b; t0 += CH) {
    const int nt = min(CH, b - t0);
    __syncthreads();                                  // the previous chunk has been consumed
    if constexpr (PF) {
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const int e = threadIdx.x + s * kScanThreads, tt = e / D, i = e % D;
        if (tt < nt) { sq[tt][i] = pq[s]; sk[tt][i] = pk[s]; sg[tt][i] = expf(pg[s]); }
      }
#pragma unroll
      for (int s = 0; s < NV; ++s) {
        const int e = threadIdx.x + s * kScanThreads;
        if (e < nt * kColsPerCta) sv[e / kColsPerCta][e % kColsPerCta] = pv[s];
      }
      if (threadIdx.x < nt) sbeta[threadIdx.x] = pbeta;
    } else {
      for (int e = threadIdx.x; e < nt * D; e += kScanThreads) {
        const int tt = e / D, i = e % D, t = t0 + tt;
        const bool in = i < p.d;
        sq[tt][i] = in ? ld(q + t * p.ldq + kh * p.d + i) : 0.f;
        sk[tt][i] = in ? ld(k + t * p.ldk + kh * p.d + i) : 0.f;
        sg[tt][i] = in ? expf(p.decay_per_head ? p.log_decay[static_cast<int64_t>(t) * p.H + h] : p.log_decay[(static_cast<int64_t>(t) * p.H + h) * p.d + i]) : 1.f;
      }
      for (int e = threadIdx.x; e < nt * kColsPerCta; e += kScanThreads) {
        const int tt = e / kColsPerCta, c = blockIdx.x * kColsPerCta + e % kColsPerCta;
        sv[tt][e % kColsPerCta] = c < p.dv ? ld(v + (t0 + tt) * p.ldv + h * p.dv + c) : 0.f;
      }
      if (threadIdx.x < nt) sbeta[threadIdx.x] = p.beta[static_cast<int64_t>(t0 + threadIdx.x) * p.H + h];
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += n_warps) {     // unit length (and the query's scale)
      float qq = 0.f, kk = 0.f;
      for (int i = lane; i < D; i += 32) { qq += sq[tt][i] * sq[tt][i]; kk += sk[tt][i] * sk[tt][i]; }
      qq = warp_sum(qq); kk = warp_sum(kk);
      const float rq = (p.unit_eps >= 0.f ? 1.0f / sqrtf(qq + p.unit_eps) : 1.0f) * p.q_scale;
      const float rk = p.unit_eps >= 0.f ? 1.0f / sqrtf(kk + p.unit_eps) : 1.0f;
      for (int i = lane; i < D; i += 32) { sq[tt][i] *= rq; sk[tt][i] *= rk; }
    }
    __syncthreads();
    if (PF && t0 + CH < b) prefetch(t0 + CH, min(CH, b - t0 - CH));
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      const int t = t0 + tt;
      const float vv = sv[tt][threadIdx.x >> 2];
      float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
      for (int e = 0; e < RP; e += 2) {
        S[e] *= sg[tt][e * kParts + part];
        acc0 = fmaf(S[e], sk[tt][e * kParts + part], acc0);
        S[e + 1] *= sg[tt][(e + 1) * kParts + part];
        acc1 = fmaf(S[e + 1], sk[tt][(e + 1) * kParts + part], acc1);
      }
      const float u = sbeta[tt] * (vv - part_sum(acc0 + acc1));
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int e = 0; e < RP; e += 2) {
        S[e] = fmaf(sk[tt][e * kParts + part], u, S[e]);
        o0 = fmaf(S[e], sq[tt][e * kParts + part], o0);
        S[e + 1] = fmaf(sk[tt][(e + 1) * kParts + part], u, S[e + 1]);
        o1 = fmaf(S[e + 1], sq[tt][(e + 1) * kParts + part], o1);
      }
      const float o = part_sum(o0 + o1);
      if (live && part == 0) p.out[(static_cast<int64_t>(t) * p.H + h) * p.dv + col] = o;
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
// mLSTM.  Same layout; the normaliser n (a d-vector) and the running maximum m are advanced by every column block of a
// head (they do not depend on the columns) and written back by the first one.
// ---------------------------------------------------------------------------------------------------------------------
template <typename T, int D, bool PF>
__global__ void __launch_bounds__(kScanThreads) mlstm_scan_kernel(MlstmArgs p) {
  constexpr int CH = ScanChunk<D>::value, RP = D / kParts;
  __shared__ float sq[CH][D], sk[CH][D], sp[CH][D];
  __shared__ float sv[CH][kColsPerCta];
  __shared__ float skeep[CH], sput[CH], sfloor[CH], sden[CH], sli[CH], slf[CH];
  constexpr int NPT = (D + kScanThreads - 1) / kScanThreads;     // normaliser entries per thread
  const int h = blockIdx.y, r = blockIdx.z;
  const int part = threadIdx.x & (kParts - 1);
  const int col = blockIdx.x * kColsPerCta + (threadIdx.x >> 2);
  const bool live = col < p.dv;
  const int a = p.cu[r], b = p.cu[r + 1];
  if (a >= b) return;
  const int64_t row = p.rows[r];
  float* state = p.state + (row * p.H + h) * p.d * p.dv;
  float* nstate = p.norm_state + (row * p.H + h) * p.d;
  float S[RP], nvec[NPT];
#pragma unroll
  for (int e = 0; e < RP; ++e) {
    const int i = e * kParts + part;
    S[e] = (live && i < p.d) ? state[static_cast<int64_t>(i) * p.dv + col] : 0.f;
  }
#pragma unroll
  for (int e = 0; e < NPT; ++e) {
    const int i = threadIdx.x + e * kScanThreads;
    nvec[e] = (i < p.d) ? nstate[i] : 0.f;
  }
  float m = p.max_state[row * p.H + h];
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, n_warps = kScanThreads >> 5;
  constexpr int NS = CH * D / kScanThreads, NV = (CH * kColsPerCta + kScanThreads - 1) / kScanThreads;
  float pq[NS], pk[NS], pv[NV], pli = 0.f, plf = 0.f;
  auto prefetch = [&](int t0, int nt) {              // the next chunk's inputs, in flight during the sequential part
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int e = threadIdx.x + s * kScanThreads, tt = e / D, i = e % D, t = t0 + tt;
      const bool in = tt < nt && i < p.d;
      pq[s] = in ? ld(q + t * p.ldq + h * p.d + i) * p.q_scale : 0.f;
      pk[s] = in ? ld(k + t * p.ldk + h * p.d + i) : 0.f;
    }
#pragma unroll
    for (int s = 0; s < NV; ++s) {
      const int e = threadIdx.x + s * kScanThreads, tt = e / kColsPerCta, c = blockIdx.x * kColsPerCta + e % kColsPerCta;
      pv[s] = (tt < nt && c < p.dv) ? ld(v + (t0 + tt) * p.ldv + h * p.dv + c) : 0.f;
    }
    if (threadIdx.x < nt) {
      pli = p.log_i[static_cast<int64_t>(t0 + threadIdx.x) * p.H + h];
      plf = p.log_f[static_cast<int64_t>(t0 + threadIdx.x) * p.H + h];
    }
  };
  if (PF) prefetch(a, min(CH, b - a));
  for (int t0 = a; t0 < b; t0 += CH) {
    const int nt = min(CH, b - t0);
    __syncthreads();                                  // the previous chunk has been consumed
    if constexpr (PF) {
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const int e = threadIdx.x + s * kScanThreads, tt = e / D, i = e % D;
        if (tt < nt) { sq[tt][i] = pq[s]; sk[tt][i] = pk[s]; }
      }
#pragma unroll
      for (int s = 0; s < NV; ++s) {
        const int e = threadIdx.x + s * kScanThreads;
        if (e < nt * kColsPerCta) sv[e / kColsPerCta][e % kColsPerCta] = pv[s];
      }
      if (threadIdx.x < nt) { sli[threadIdx.x] = pli; slf[threadIdx.x] = plf; }
    } else {
      for (int e = threadIdx.x; e < nt * D; e += kScanThreads) {
        const int tt = e / D, i = e % D, t = t0 + tt;
        const bool in = i < p.d;
        sq[tt][i] = in ? ld(q + t * p.ldq + h * p.d + i) * p.q_scale : 0.f;
        sk[tt][i] = in ? ld(k + t * p.ldk + h * p.d + i) : 0.f;
      }
      for (int e = threadIdx.x; e < nt * kColsPerCta; e += kScanThreads) {
        const int tt = e / kColsPerCta, c = blockIdx.x * kColsPerCta + e % kColsPerCta;
        sv[tt][e % kColsPerCta] = c < p.dv ? ld(v + (t0 + tt) * p.ldv + h * p.dv + c) : 0.f;
      }
      if (threadIdx.x < nt) {
        sli[threadIdx.x] = p.log_i[static_cast<int64_t>(t0 + threadIdx.x) * p.H + h];
        slf[threadIdx.x] = p.log_f[static_cast<int64_t>(t0 + threadIdx.x) * p.H + h];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {                          // the gate recurrence is scalar: one thread walks the chunk
      float mm = m;
      for (int tt = 0; tt < nt; ++tt) {
        const float li = sli[tt], lf = slf[tt];
        const float m_new = fmaxf(lf + mm, li);
        skeep[tt] = expf(lf + mm - m_new);
        sput[tt] = expf(li - m_new);
        sfloor[tt] = expf(-m_new);
        mm = m_new;
      }
      sden[0] = mm;
    }
    __syncthreads();
    m = sden[0];
    // normaliser: n <- keep n + put k, and the products n_i q_i of every token of the chunk
    for (int tt = 0; tt < nt; ++tt) {
#pragma unroll
      for (int e = 0; e < NPT; ++e) {
        const int i = threadIdx.x + e * kScanThreads;
        if (i < D) {
          nvec[e] = skeep[tt] * nvec[e] + sput[tt] * sk[tt][i];
          sp[tt][i] = nvec[e] * sq[tt][i];
        }
      }
    }
    __syncthreads();
    for (int tt = warp; tt < nt; tt += n_warps) {
      float s = 0.f;
      for (int i = lane; i < D; i += 32) s += sp[tt][i];
      s = warp_sum(s);
      if (lane == 0) sden[tt] = fmaxf(fabsf(s), sfloor[tt]) + p.denom_eps;
    }
    __syncthreads();
    if (PF && t0 + CH < b) prefetch(t0 + CH, min(CH, b - t0 - CH));
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      const int t = t0 + tt;
      const float pv = sput[tt] * sv[tt][threadIdx.x >> 2];
      const float keep = skeep[tt];
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int e = 0; e < RP; e += 2) {
        S[e] = fmaf(keep, S[e], sk[tt][e * kParts + part] * pv);
        o0 = fmaf(S[e], sq[tt][e * kParts + part], o0);
        S[e + 1] = fmaf(keep, S[e + 1], sk[tt][(e + 1) * kParts + part] * pv);
        o1 = fmaf(S[e + 1], sq[tt][(e + 1) * kParts + part], o1);
      }
      const float o = part_sum(o0 + o1);
      if (live && part == 0) p.out[(static_cast<int64_t>(t) * p.H + h) * p.dv + col] = o / sden[tt];
    }
  }
  if (live) {
#pragma unroll
    for (int e = 0; e < RP; ++e) {
      const int i = e * kParts + part;
      if (i < p.d) state[static_cast<int64_t>(i) * p.dv + col] = S[e];
    }
  }
  if (blockIdx.x == 0) {
#pragma unroll
    for (int e = 0; e < NPT; ++e) {
      const int i = threadIdx.x + e * kScanThreads;
      if (i < p.d) nstate[i] = nvec[e];
    }
    if (threadIdx.x == 0) p.max_state[row * p.H + h] = m;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// latent attention over paged latents.  grid (tokens, head blocks, key splits).  The CTA stages tiles of kKeyTile latents
// in shared memory once for all of its heads; every warp owns HGW heads (queries and accumulators in registers, the latent
// dimension spread over the lanes) and walks all keys of the CTA's range with an online softmax, kKeyBatch keys at a time so
// that the score reductions overlap.  With more than one split (few query tokens, long contexts) every warp leaves (max, sum,
// weighted sum) in a workspace and a second kernel merges the splits.
// ---------------------------------------------------------------------------------------------------------------------
constexpr int kAttnWarps = 8;
constexpr int kKeyTile = 16;
constexpr int kKeyBatch = 4;

template <typename T, int RPL, int HGW>
__global__ void __launch_bounds__(kAttnWarps * 32) latent_attention_kernel(LatentAttnArgs p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* tile = reinterpret_cast<T*>(smem_raw);          // [kKeyTile][r]
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h0 = (blockIdx.y * kAttnWarps + warp) * HGW;
  const int nh = max(0, min(HGW, p.H - h0));
  const int r = p.r, len = p.tok_len[t];
  const int per_split = (len + p.n_splits - 1) / p.n_splits;
  const int key_lo = blockIdx.z * per_split, key_hi = min(len, key_lo + per_split);
  const int* table = p.block_table + static_cast<int64_t>(p.tok_req[t]) * p.max_blocks;
  const T* cache = static_cast<const T*>(p.cache);
  float qv[HGW][RPL], acc[HGW][RPL], mx[HGW], l[HGW];
#pragma unroll
  for (int g = 0; g < HGW; ++g) {
    mx[g] = -INFINITY; l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < RPL; ++e) {
      const int i = lane + 32 * e;
      qv[g][e] = (g < nh && i < r) ? ld(static_cast<const T*>(p.q) + (static_cast<int64_t>(t) * p.H + h0 + g) * r + i) * p.scale : 0.f;
      acc[g][e] = 0.f;
    }
  }
  constexpr int VEC = 16 / sizeof(T);
  for (int tile_lo = key_lo; tile_lo < key_hi; tile_lo += kKeyTile) {
    const int nk = min(kKeyTile, key_hi - tile_lo);
    __syncthreads();                                  // the previous tile has been consumed
    for (int j = warp; j < nk; j += kAttnWarps) {
      const int key = tile_lo + j;
      const T* src = cache + (static_cast<int64_t>(table[key / p.block_size]) * p.block_size + key % p.block_size) * r;
      if (p.vec_ok) {
        for (int i = lane * VEC; i < r; i += 32 * VEC)
          *reinterpret_cast<uint4*>(tile + j * r + i) = *reinterpret_cast<const uint4*>(src + i);
      } else {
        for (int i = lane; i < r; i += 32) tile[j * r + i] = src[i];
      }
    }
    __syncthreads();
    if (nh == 0) continue;
    for (int j0 = 0; j0 < nk; j0 += kKeyBatch) {
      float sc[HGW][kKeyBatch];
#pragma unroll
      for (int g = 0; g < HGW; ++g)
#pragma unroll
        for (int kb = 0; kb < kKeyBatch; ++kb) sc[g][kb] = 0.f;
#pragma unroll
      for (int kb = 0; kb < kKeyBatch; ++kb) {
        if (j0 + kb < nk) {
#pragma unroll
          for (int e = 0; e < RPL; ++e) {
            const int i = lane + 32 * e;
            const float c = i < r ? ld(tile + (j0 + kb) * r + i) : 0.f;
#pragma unroll
            for (int g = 0; g < HGW; ++g) sc[g][kb] = fmaf(qv[g][e], c, sc[g][kb]);
          }
        }
      }
#pragma unroll
      for (int g = 0; g < HGW; ++g)
#pragma unroll
        for (int kb = 0; kb < kKeyBatch; ++kb) sc[g][kb] = (j0 + kb < nk) ? warp_sum(sc[g][kb]) : -INFINITY;
      float corr[HGW];
#pragma unroll
      for (int g = 0; g < HGW; ++g) {
        float m_new = mx[g];
#pragma unroll
        for (int kb = 0; kb < kKeyBatch; ++kb) m_new = fmaxf(m_new, sc[g][kb]);
        corr[g] = expf(mx[g] - m_new);
        float wsum = 0.f;
#pragma unroll
        for (int kb = 0; kb < kKeyBatch; ++kb) { sc[g][kb] = expf(sc[g][kb] - m_new); wsum += sc[g][kb]; }
        l[g] = l[g] * corr[g] + wsum;
        mx[g] = m_new;
      }
#pragma unroll
      for (int e = 0; e < RPL; ++e) {
        const int i = lane + 32 * e;
        float c[kKeyBatch];
#pragma unroll
        for (int kb = 0; kb < kKeyBatch; ++kb) c[kb] = (i < r && j0 + kb < nk) ? ld(tile + (j0 + kb) * r + i) : 0.f;
#pragma unroll
        for (int g = 0; g < HGW; ++g) {
          float a = acc[g][e] * corr[g];
#pragma unroll
          for (int kb = 0; kb < kKeyBatch; ++kb) a = fmaf(sc[g][kb], c[kb], a);
          acc[g][e] = a;
        }
      }
    }
  }
#pragma unroll
  for (int g = 0; g < HGW; ++g) {
    if (g >= nh) continue;
    const int64_t row = static_cast<int64_t>(t) * p.H + h0 + g;
    if (p.n_splits == 1) {
      const float inv = 1.0f / l[g];
#pragma unroll
      for (int e = 0; e < RPL; ++e) {
        const int i = lane + 32 * e;
        if (i < r) p.out[row * r + i] = acc[g][e] * inv;
      }
    } else {
      float* ws = p.ws + (row * p.n_splits + blockIdx.z) * (r + 2);
      if (lane == 0) { ws[0] = mx[g]; ws[1] = l[g]; }
#pragma unroll
      for (int e = 0; e < RPL; ++e) {
        const int i = lane + 32 * e;
        if (i < r) ws[2 + i] = acc[g][e];
      }
    }
  }
}

// one warp per (token, head): merge the splits' (max, sum, weighted sum)
__global__ void latent_attention_merge_kernel(const float* __restrict__ ws, float* __restrict__ out, int n_rows, int r, int n_splits) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int lane = threadIdx.x & 31;
  const float* base = ws + static_cast<int64_t>(row) * n_splits * (r + 2);
  float m_all = -INFINITY;
  for (int z = 0; z < n_splits; ++z) m_all = fmaxf(m_all, base[z * (r + 2)]);
  float den = 0.f;
  for (int z = 0; z < n_splits; ++z) {
    const float mz = base[z * (r + 2)];
    den += (mz == -INFINITY ? 0.f : expf(mz - m_all)) * base[z * (r + 2) + 1];
  }
  for (int i = lane; i < r; i += 32) {
    float num = 0.f;
    for (int z = 0; z < n_splits; ++z) {
      const float mz = base[z * (r + 2)];
      num += (mz == -INFINITY ? 0.f : expf(mz - m_all)) * base[z * (r + 2) + 2 + i];
    }
    out[static_cast<int64_t>(row) * r + i] = num / den;
  }
}

// ---------------------------------------------------------------------------------------------------------------------
// router: one warp per token
// ---------------------------------------------------------------------------------------------------------------------
__global__ void group_limited_router_kernel(const float* __restrict__ logits, float* __restrict__ probs, bool* __restrict__ rmap,
                                            int n_tok, int E, int topk, int G, int keep, int renorm) {
  extern __shared__ float smem[];                   // per warp: scores [E], group best [G]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * (blockDim.x >> 5) + warp;
  if (t >= n_tok) return;
  float* s = smem + static_cast<int64_t>(warp) * (E + G);
  float* gbest = s + E;
  const float* z = logits + static_cast<int64_t>(t) * E;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = warp_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) { const float v = expf(z[e] - mx); s[e] = v; sum += v; }
  sum = warp_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) s[e] = s[e] / sum;
  __syncwarp();
  const int per = E / G;
  for (int g = lane; g < G; g += 32) {
    float b = -1.f;
    for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, s[e]);
    gbest[g] = b;
  }
  __syncwarp();
  // drop all but the `keep` best groups: repeatedly take the best remaining group and mark it (score + 2 > 1)
  for (int it = 0; it < keep; ++it) {
    float bv = -1.f; int bi = 0x7fffffff;
    for (int g = lane; g < G; g += 32) {
      const float v = gbest[g];
      if (v <= 1.5f && (v > bv || (v == bv && g < bi))) { bv = v; bi = g; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0 && bi < G) gbest[bi] += 2.f;
    __syncwarp();
  }
  float wsum = 0.f;
  int chosen[32];                                   // topk <= 32 (checked on the host)
  for (int it = 0; it < topk; ++it) {
    float bv = -1.f; int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = s[e];
      if (v >= 0.f && gbest[e / per] > 1.5f && (v > bv || (v == bv && e < bi))) { bv = v; bi = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o); const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    chosen[it] = bi;
    if (bi < E) {
      wsum += bv;
      if (lane == 0) { probs[static_cast<int64_t>(t) * E + bi] = bv; s[bi] = -1.f; }
    }
    __syncwarp();
  }
  if (lane == 0) {
    const float inv = renorm ? 1.0f / (wsum + 1e-20f) : 1.0f;
    for (int it = 0; it < topk; ++it)
      if (chosen[it] < E) {
        probs[static_cast<int64_t>(t) * E + chosen[it]] *= inv;
        rmap[static_cast<int64_t>(t) * E + chosen[it]] = true;
      }
  }
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------------------------------------
#define SEQ_DISPATCH_T(is_bf16, ...)                      \
  if (is_bf16) { using T = __nv_bfloat16; __VA_ARGS__; }  \
  else { using T = float; __VA_ARGS__; }

void add_rms_norm(float* x, const void* delta, const void* w, void* y, int rows, int cols, float eps, float w_off, bool bf16,
                  cudaStream_t s) {
  if (rows == 0) return;
  SEQ_DISPATCH_T(bf16, add_rms_norm_kernel<T><<<rows, 256, cols * sizeof(float), s>>>(
                           x, static_cast<const T*>(delta), static_cast<const T*>(w), static_cast<T*>(y), cols, eps, w_off));
}

void gated_head_rms_norm(const float* o, const void* w, const void* gate, int64_t ldg, void* y, int n_tok, int H, int dv,
                         bool w_per_head, float eps, bool silu, bool bf16, cudaStream_t s) {
  const int rows = n_tok * H;
  if (rows == 0) return;
  SEQ_DISPATCH_T(bf16, gated_head_rms_norm_kernel<T><<<(rows + 3) / 4, 128, 0, s>>>(
                           o, static_cast<const T*>(w), static_cast<const T*>(gate), ldg, static_cast<T*>(y), rows, H, dv,
                           w_per_head ? 1 : 0, eps, silu ? 1 : 0));
}

template <typename T, int TAPS>
static void launch_conv_run(const void* x, int64_t ldx, const void* w, const void* bias, const int* cu, const int* rows,
                            const void* window, void* y,
                            int R, int C, int max_len, int silu, cudaStream_t s) {
  dim3 grid((C / 2 + 127) / 128, (max_len + kConvRun - 1) / kConvRun, R);
  causal_conv_silu_run_kernel<T, TAPS><<<grid, 128, 0, s>>>(static_cast<const T*>(x), ldx, static_cast<const T*>(w),
                                                            static_cast<const T*>(bias), cu, rows,
                                                            static_cast<const T*>(window), static_cast<T*>(y), C, silu);
}

void causal_conv_silu(const void* x, int64_t ldx, const void* w, const void* bias, const int* cu, const int* rows, const int* tok_seq,
                      void* window,
                      void* y, int n_tok, int R, int C, int taps, int max_len, bool silu, bool residual, bool bf16, cudaStream_t s) {
  if (n_tok == 0) return;
  const int act = (silu ? 1 : 0) | (residual ? 2 : 0);
  const int64_t n = static_cast<int64_t>(n_tok) * C;
  // the paired kernel needs even channel counts and strides, 4- / 8-byte aligned bases, and a grid within the launch limits
  const size_t pair_bytes = bf16 ? 4 : 8;
  const bool paired = taps >= 2 && taps <= 4 && C % 2 == 0 && ldx % 2 == 0 && reinterpret_cast<uintptr_t>(x) % pair_bytes == 0 &&
                      reinterpret_cast<uintptr_t>(y) % pair_bytes == 0 && reinterpret_cast<uintptr_t>(window) % pair_bytes == 0 &&
                      max_len > 0 && (max_len + kConvRun - 1) / kConvRun <= 65535 && R <= 65535;
  SEQ_DISPATCH_T(bf16, {
    if (paired && taps == 2) launch_conv_run<T, 2>(x, ldx, w, bias, cu, rows, window, y, R, C, max_len, act, s);
    else if (paired && taps == 3) launch_conv_run<T, 3>(x, ldx, w, bias, cu, rows, window, y, R, C, max_len, act, s);
    else if (paired && taps == 4) launch_conv_run<T, 4>(x, ldx, w, bias, cu, rows, window, y, R, C, max_len, act, s);
    else causal_conv_silu_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(
        static_cast<const T*>(x), ldx, static_cast<const T*>(w), static_cast<const T*>(bias), cu, rows, tok_seq,
        static_cast<const T*>(window),
        static_cast<T*>(y), n_tok, C, taps, act);
    if (taps > 1)
      conv_window_update_kernel<T><<<(R * C + 255) / 256, 256, 0, s>>>(static_cast<const T*>(x), ldx, cu, rows,
                                                                        static_cast<T*>(window), R, C, taps);
  });
}

template <typename T>
static bool launch_delta(const DeltaArgs& p, dim3 grid, cudaStream_t s) {
#define SEQ_DELTA(DD)                                                                                   \
  if (p.max_len > ScanChunk<DD>::value) delta_rule_scan_kernel<T, DD, true><<<grid, kScanThreads, 0, s>>>(p); \
  else delta_rule_scan_kernel<T, DD, false><<<grid, kScanThreads, 0, s>>>(p)
  if (p.d <= 32) { SEQ_DELTA(32); }
  else if (p.d <= 64) { SEQ_DELTA(64); }
  else if (p.d <= 128) { SEQ_DELTA(128); }
  else if (p.d <= 256) { SEQ_DELTA(256); }
  else return false;
#undef SEQ_DELTA
  return true;
}

bool delta_rule_scan(const DeltaArgs& p, int R, bool bf16, cudaStream_t s) {
  if (R == 0) return true;
  dim3 grid((p.dv + kColsPerCta - 1) / kColsPerCta, p.H, R);
  return bf16 ? launch_delta<__nv_bfloat16>(p, grid, s) : launch_delta<float>(p, grid, s);
}

template <typename T>
static bool launch_mlstm(const MlstmArgs& p, dim3 grid, cudaStream_t s) {
#define SEQ_MLSTM(DD)                                                                              \
  if (p.max_len > ScanChunk<DD>::value) mlstm_scan_kernel<T, DD, true><<<grid, kScanThreads, 0, s>>>(p); \
  else mlstm_scan_kernel<T, DD, false><<<grid, kScanThreads, 0, s>>>(p)
  if (p.d <= 32) { SEQ_MLSTM(32); }
  else if (p.d <= 64) { SEQ_MLSTM(64); }
  else if (p.d <= 128) { SEQ_MLSTM(128); }
  else if (p.d <= 256) { SEQ_MLSTM(256); }
  else return false;
#undef SEQ_MLSTM
  return true;
}

bool mlstm_scan(const MlstmArgs& p, int R, bool bf16, cudaStream_t s) {
  if (R == 0) return true;
  dim3 grid((p.dv + kColsPerCta - 1) / kColsPerCta, p.H, R);
  return bf16 ? launch_mlstm<__nv_bfloat16>(p, grid, s) : launch_mlstm<float>(p, grid, s);
}

template <typename T, int RPL, int HGW>
static bool launch_attn(const LatentAttnArgs& p, int n_tok, cudaStream_t s) {
  const size_t smem = static_cast<size_t>(kKeyTile) * p.r * sizeof(T);
  auto kern = latent_attention_kernel<T, RPL, HGW>;
  if (smem > 48 * 1024 && cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess)
    return false;
  dim3 grid(n_tok, (p.H + kAttnWarps * HGW - 1) / (kAttnWarps * HGW), p.n_splits);
  kern<<<grid, kAttnWarps * 32, smem, s>>>(p);
  if (p.n_splits > 1) {
    const int rows = n_tok * p.H;
    latent_attention_merge_kernel<<<(rows + 3) / 4, 128, 0, s>>>(p.ws, p.out, rows, p.r, p.n_splits);
  }
  return true;
}

// latent entries per lane (a power of two >= r / 32) and heads per warp: as many as fit 32 accumulators per lane, but no more
// than it takes to spread the heads over the CTA's warps
static void attn_shape(int H, int r, int* rpl, int* hgw) {
  int e = 2;
  while (e * 32 < r) e *= 2;
  int g = 1;
  while (g < 8 && g * 2 * e <= 32 && kAttnWarps * g < H) g *= 2;
  *rpl = e; *hgw = g;
}

template <typename T, int RPL>
static bool dispatch_attn_hgw(const LatentAttnArgs& p, int hgw, int n_tok, cudaStream_t s) {
  if (hgw == 1) return launch_attn<T, RPL, 1>(p, n_tok, s);
  if constexpr (RPL <= 16) { if (hgw == 2) return launch_attn<T, RPL, 2>(p, n_tok, s); }
  if constexpr (RPL <= 8) { if (hgw == 4) return launch_attn<T, RPL, 4>(p, n_tok, s); }
  if constexpr (RPL <= 4) { if (hgw == 8) return launch_attn<T, RPL, 8>(p, n_tok, s); }
  return false;
}

template <typename T>
static bool dispatch_attn(const LatentAttnArgs& p, int n_tok, cudaStream_t s) {
  int rpl, hgw;
  attn_shape(p.H, p.r, &rpl, &hgw);
  switch (rpl) {
    case 2: return dispatch_attn_hgw<T, 2>(p, hgw, n_tok, s);
    case 4: return dispatch_attn_hgw<T, 4>(p, hgw, n_tok, s);
    case 8: return dispatch_attn_hgw<T, 8>(p, hgw, n_tok, s);
    case 16: return dispatch_attn_hgw<T, 16>(p, hgw, n_tok, s);
    case 32: return dispatch_attn_hgw<T, 32>(p, hgw, n_tok, s);
    default: return false;
  }
}

int latent_attention_splits(int H, int r, int n_tok, int max_len) {
  int rpl, hgw;
  attn_shape(H, r, &rpl, &hgw);
  const int64_t ctas = static_cast<int64_t>(n_tok) * ((H + kAttnWarps * hgw - 1) / (kAttnWarps * hgw));
  if (ctas >= 2 * 148 || max_len < 8 * kKeyTile) return 1;
  const int64_t want = (4 * 148 + ctas - 1) / ctas;
  return static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(want, 64), max_len / (4 * kKeyTile))));
}

bool latent_attention_paged(const LatentAttnArgs& p, int n_tok, bool bf16, cudaStream_t s) {
  if (n_tok == 0) return true;
  return bf16 ? dispatch_attn<__nv_bfloat16>(p, n_tok, s) : dispatch_attn<float>(p, n_tok, s);
}

bool group_limited_router(const float* logits, float* probs, bool* rmap, int n_tok, int E, int topk, int G, int keep, bool renorm,
                          cudaStream_t s) {
  if (n_tok == 0) return true;
  if (topk > 32 || G <= 0 || E % G != 0) return false;
  const int warps = 4;
  const size_t smem = static_cast<size_t>(warps) * (E + G) * sizeof(float);
  if (smem > 48 * 1024) return false;
  group_limited_router_kernel<<<(n_tok + warps - 1) / warps, warps * 32, smem, s>>>(logits, probs, rmap, n_tok, E, topk, G, keep,
                                                                                   renorm ? 1 : 0);
  return true;
}

}  // namespace b200seq
