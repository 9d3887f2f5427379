// Sequence-mixing kernels (sm_100a), third part: retention scan with rotary positions applied on the way in, the
// polynomial-of-norms activation, and the tanh-GELU gate times a per-token vector.
//
// Conventions as in seqmix.cu: activations are `T` (float or __nv_bfloat16); angles, rotated vectors, statistics and the
// recurrent state are fp32.  `cu[R + 1]` holds the sequence boundaries of the packed batch, `rows[R]` the state row of every
// sequence.
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

// ---------------------------------------------------------------------------------------------------------------------
// retention: S <- decay_h S + (k_scale rot(k)) v^T;  o = S^T rot(q).  grid (column blocks, heads, sequences).  The layout of
// the gated delta-rule scan: a column of S is shared by kParts adjacent lanes, lane `part` keeps rows part, part + kParts,
// ... in registers; q, k and the value columns of a chunk of tokens are staged in shared memory as fp32, where q and k are
// turned by their token's position (dimension i with i + n_rot) before the sequential part; one reduction over the key
// dimension per token ends in two shuffles.
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
__global__ void __launch_bounds__(kScanThreads) retention_scan_kernel(RetentionArgs p) {
  constexpr int CH = ScanChunk<D>::value, RP = D / kParts;
  __shared__ float sq[CH][D], sk[CH][D];
  __shared__ float sv[CH][kColsPerCta];
  __shared__ float spos[CH];
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
  const float decay = p.decay[h], ks = p.k_scale;
  const int n_rot = p.n_rot, rot_end = 2 * n_rot;
  const T* q = static_cast<const T*>(p.q);
  const T* k = static_cast<const T*>(p.k);
  const T* v = static_cast<const T*>(p.v);
  // With PF (sequences longer than a chunk) the next chunk's inputs are fetched into registers before the sequential part of
  // the current one; without it (decoding) a chunk is fetched when its turn comes, which keeps the registers free.
  constexpr int NS = CH * D / kScanThreads, NV = (CH * kColsPerCta + kScanThreads - 1) / kScanThreads;
  float pq[NS], pk[NS], pv[NV], ppos = 0.f;
  auto prefetch = [&](int t0, int nt) {
#pragma unroll
    for (int s = 0; s < NS; ++s) {
      const int e = threadIdx.x + s * kScanThreads, tt = e / D, i = e % D, t = t0 + tt;
      const bool in = tt < nt && i < p.d;
      pq[s] = in ? ld(q + t * p.ldq + h * p.d + i) : 0.f;
      pk[s] = in ? ld(k + t * p.ldk + h * p.d + i) : 0.f;
    }
#pragma unroll
    for (int s = 0; s < NV; ++s) {
      const int e = threadIdx.x + s * kScanThreads, tt = e / kColsPerCta, c = blockIdx.x * kColsPerCta + e % kColsPerCta;
      pv[s] = (tt < nt && c < p.dv) ? ld(v + (t0 + tt) * p.ldv + h * p.dv + c) : 0.f;
    }
    if (n_rot > 0 && threadIdx.x < nt) ppos = static_cast<float>(p.positions[t0 + threadIdx.x]);
  };
  if (PF) prefetch(a, min(CH, b - a));
  for (int t0 = a; t0 < b; t0 += CH) {
    const int nt = min(CH, b - t0);
    __syncthreads();                                  // the previous chunk has been consumed
    if constexpr (PF) {
#pragma unroll
      for (int s = 0; s < NS; ++s) {
        const int e = threadIdx.x + s * kScanThreads, tt = e / D, i = e % D;
        if (tt < nt) { sq[tt][i] = pq[s]; sk[tt][i] = i >= rot_end ? pk[s] * ks : pk[s]; }
      }
#pragma unroll
      for (int s = 0; s < NV; ++s) {
        const int e = threadIdx.x + s * kScanThreads;
        if (e < nt * kColsPerCta) sv[e / kColsPerCta][e % kColsPerCta] = pv[s];
      }
      if (n_rot > 0 && threadIdx.x < nt) spos[threadIdx.x] = ppos;
    } else {
      for (int e = threadIdx.x; e < nt * D; e += kScanThreads) {
        const int tt = e / D, i = e % D, t = t0 + tt;
        const bool in = i < p.d;
        sq[tt][i] = in ? ld(q + t * p.ldq + h * p.d + i) : 0.f;
        const float kv = in ? ld(k + t * p.ldk + h * p.d + i) : 0.f;
        sk[tt][i] = i >= rot_end ? kv * ks : kv;
      }
      for (int e = threadIdx.x; e < nt * kColsPerCta; e += kScanThreads) {
        const int tt = e / kColsPerCta, c = blockIdx.x * kColsPerCta + e % kColsPerCta;
        sv[tt][e % kColsPerCta] = c < p.dv ? ld(v + (t0 + tt) * p.ldv + h * p.dv + c) : 0.f;
      }
      if (n_rot > 0 && threadIdx.x < nt) spos[threadIdx.x] = static_cast<float>(p.positions[t0 + threadIdx.x]);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < nt * n_rot; e += kScanThreads) {       // turn the pairs (i, i + n_rot) of q and k
      const int tt = e / n_rot, i = e - tt * n_rot;
      float sn, cs;
      sincosf(spos[tt] * p.inv_freq[i], &sn, &cs);
      const float qu = sq[tt][i], qw = sq[tt][i + n_rot], ku = sk[tt][i], kw = sk[tt][i + n_rot];
      sq[tt][i] = qu * cs - qw * sn;
      sq[tt][i + n_rot] = qw * cs + qu * sn;
      sk[tt][i] = (ku * cs - kw * sn) * ks;
      sk[tt][i + n_rot] = (kw * cs + ku * sn) * ks;
    }
    if (n_rot > 0) __syncthreads();
    if (PF && t0 + CH < b) prefetch(t0 + CH, min(CH, b - t0 - CH));
#pragma unroll 1
    for (int tt = 0; tt < nt; ++tt) {
      const float vv = sv[tt][threadIdx.x >> 2];
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int e = 0; e < RP; e += 2) {
        S[e] = fmaf(decay, S[e], sk[tt][e * kParts + part] * vv);
        o0 = fmaf(S[e], sq[tt][e * kParts + part], o0);
        S[e + 1] = fmaf(decay, S[e + 1], sk[tt][(e + 1) * kParts + part] * vv);
        o1 = fmaf(S[e + 1], sq[tt][(e + 1) * kParts + part], o1);
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
// y = a N(z) + b N(z^2) + c N(z^3) + e, N(u) = u / sqrt(mean(u^2) + eps): one CTA per row, two passes over the row (the
// second one finds it in cache); V elements per access.
// ---------------------------------------------------------------------------------------------------------------------
template <typename T, int V> struct RowVec;
template <> struct RowVec<float, 1> {
  static __device__ __forceinline__ void load(const float* p, float* o) { o[0] = *p; }
  static __device__ __forceinline__ void store(float* p, const float* o) { *p = o[0]; }
};
template <> struct RowVec<__nv_bfloat16, 1> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) { o[0] = __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* o) { *p = __float2bfloat16_rn(o[0]); }
};
template <> struct RowVec<float, 4> {
  static __device__ __forceinline__ void load(const float* p, float* o) {
    const float4 r = *reinterpret_cast<const float4*>(p);
    o[0] = r.x; o[1] = r.y; o[2] = r.z; o[3] = r.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* o) { *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]); }
};
template <> struct RowVec<__nv_bfloat16, 8> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* o) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h2[e]); o[2 * e] = f.x; o[2 * e + 1] = f.y; }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* o) {
    uint4 r;
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
    for (int e = 0; e < 4; ++e) h2[e] = __floats2bfloat162_rn(o[2 * e], o[2 * e + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
};

template <typename T, int V>
__global__ void __launch_bounds__(256) poly_norm_kernel(const T* __restrict__ z, int64_t ldz, const float* __restrict__ coef, T* __restrict__ y,
                                                        int cols, float eps) {
  __shared__ float red[3][8];
  const T* src = z + static_cast<int64_t>(blockIdx.x) * ldz;
  T* dst = y + static_cast<int64_t>(blockIdx.x) * cols;
  float s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (int c = threadIdx.x * V; c < cols; c += blockDim.x * V) {
    float x[V];
    RowVec<T, V>::load(src + c, x);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const float x2 = x[e] * x[e];
      s1 += x2; s2 = fmaf(x2, x2, s2); s3 = fmaf(x2 * x2, x2, s3);
    }
  }
  s1 = warp_sum(s1); s2 = warp_sum(s2); s3 = warp_sum(s3);
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s1; red[1][threadIdx.x >> 5] = s2; red[2][threadIdx.x >> 5] = s3; }
  __syncthreads();
  float t1 = 0.f, t2 = 0.f, t3 = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { t1 += red[0][i]; t2 += red[1][i]; t3 += red[2][i]; }
  const float inv_n = 1.0f / static_cast<float>(cols);
  const float a = coef[0] / sqrtf(t1 * inv_n + eps), b = coef[1] / sqrtf(t2 * inv_n + eps), c3 = coef[2] / sqrtf(t3 * inv_n + eps);
  const float e0 = coef[3];
  for (int c = threadIdx.x * V; c < cols; c += blockDim.x * V) {
    float x[V];
    RowVec<T, V>::load(src + c, x);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      const float x1 = x[e], x2 = x1 * x1;
      x[e] = fmaf(a, x1, fmaf(b, x2, fmaf(c3, x2 * x1, e0)));
    }
    RowVec<T, V>::store(dst + c, x);
  }
}

template <typename T>
__global__ void gelu_mul_kernel(const T* __restrict__ g, int64_t ldg, const T* __restrict__ e, int64_t lde, T* __restrict__ y,
                                int64_t rows, int cols) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= rows * cols) return;
  const int64_t r = idx / cols;
  const int c = static_cast<int>(idx - r * cols);
  const float zv = ld(g + r * ldg + c);
  const float act = 0.5f * zv * (1.0f + tanhf(0.7978845608028654f * (zv + 0.044715f * zv * zv * zv)));
  st(y + idx, act * ld(e + r * lde + c));
}

// log_decay = -exp(A_log[head]) * softplus(a + dt_bias), beta = sigmoid(b): the gates of the delta rule from the projections'
// pre-activations, fp32 out.  C decay channels per row, C / H per head.
template <typename T>
__global__ void decay_gates_kernel(const T* __restrict__ a, int64_t lda, const T* __restrict__ b, int64_t ldb, const T* __restrict__ A_log,
                                   const T* __restrict__ dt_bias, float* __restrict__ log_decay, float* __restrict__ beta, int64_t rows,
                                   int C, int H) {
  const int64_t idx = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per = C + H;                              // a row's decay channels, then its betas
  if (idx >= rows * per) return;
  const int64_t r = idx / per;
  const int c = static_cast<int>(idx - r * per);
  if (c < C) {
    const float z = ld(a + r * lda + c) + ld(dt_bias + c);
    const float sp = z > 20.f ? z : log1pf(expf(z));
    log_decay[r * C + c] = -expf(ld(A_log + c / (C / H))) * sp;
  } else {
    beta[r * H + (c - C)] = sigmoidf_(ld(b + r * ldb + (c - C)));
  }
}

template <typename T>
static bool launch_retention(const RetentionArgs& p, dim3 grid, cudaStream_t s) {
#define SEQ_RET(DD)                                                                                       \
  if (p.max_len > ScanChunk<DD>::value) retention_scan_kernel<T, DD, true><<<grid, kScanThreads, 0, s>>>(p); \
  else retention_scan_kernel<T, DD, false><<<grid, kScanThreads, 0, s>>>(p)
  if (p.d <= 32) { SEQ_RET(32); }
  else if (p.d <= 64) { SEQ_RET(64); }
  else if (p.d <= 128) { SEQ_RET(128); }
  else if (p.d <= 256) { SEQ_RET(256); }
  else return false;
#undef SEQ_RET
  return true;
}

}  // namespace

bool retention_scan(const RetentionArgs& p, int R, bool bf16, cudaStream_t s) {
  if (R == 0) return true;
  if (R > 65535 || p.H > 65535) return false;
  dim3 grid((p.dv + kColsPerCta - 1) / kColsPerCta, p.H, R);
  SEQ_DISPATCH_T(bf16, return launch_retention<T>(p, grid, s));
}

bool poly_norm(const void* z, int64_t ldz, const float* coef, void* y, int64_t rows, int cols, float eps, bool bf16, cudaStream_t s) {
  if (rows == 0 || cols == 0) return true;
  if (rows > 2147483647LL) return false;
  const unsigned grid = static_cast<unsigned>(rows);
  if (bf16) {
    using T = __nv_bfloat16;
    const bool vec = cols % 8 == 0 && ldz % 8 == 0 && reinterpret_cast<uintptr_t>(z) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
    if (vec) poly_norm_kernel<T, 8><<<grid, 256, 0, s>>>(static_cast<const T*>(z), ldz, coef, static_cast<T*>(y), cols, eps);
    else poly_norm_kernel<T, 1><<<grid, 256, 0, s>>>(static_cast<const T*>(z), ldz, coef, static_cast<T*>(y), cols, eps);
  } else {
    const bool vec = cols % 4 == 0 && ldz % 4 == 0 && reinterpret_cast<uintptr_t>(z) % 16 == 0 && reinterpret_cast<uintptr_t>(y) % 16 == 0;
    if (vec) poly_norm_kernel<float, 4><<<grid, 256, 0, s>>>(static_cast<const float*>(z), ldz, coef, static_cast<float*>(y), cols, eps);
    else poly_norm_kernel<float, 1><<<grid, 256, 0, s>>>(static_cast<const float*>(z), ldz, coef, static_cast<float*>(y), cols, eps);
  }
  return true;
}

void decay_gates(const void* a, int64_t lda, const void* b, int64_t ldb, const void* A_log, const void* dt_bias, float* log_decay, float* beta,
                 int64_t rows, int C, int H, bool bf16, cudaStream_t s) {
  const int64_t n = rows * (C + H);
  if (n == 0) return;
  SEQ_DISPATCH_T(bf16, decay_gates_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(
                           static_cast<const T*>(a), lda, static_cast<const T*>(b), ldb, static_cast<const T*>(A_log),
                           static_cast<const T*>(dt_bias), log_decay, beta, rows, C, H));
}

void gelu_mul(const void* g, int64_t ldg, const void* e, int64_t lde, void* y, int64_t rows, int cols, bool bf16, cudaStream_t s) {
  const int64_t n = rows * cols;
  if (n == 0) return;
  SEQ_DISPATCH_T(bf16, gelu_mul_kernel<T><<<static_cast<unsigned>((n + 255) / 256), 256, 0, s>>>(
                           static_cast<const T*>(g), ldg, static_cast<const T*>(e), lde, static_cast<T*>(y), rows, cols));
}

}  // namespace b200seq
