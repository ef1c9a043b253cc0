// Clustering in the rank-32 space: exact nearest-centroid assignment, stable
// grouping of rows by label, deterministic centroid updates, cluster-major V
// with per-cluster value sums, and the row gather used for K.
//
// Replaces the reference's kmeans_maintain extension
// (token2tile/operator/kernels/kmeans_maintain/src/kernels.cu) and its Triton
// helpers fast_assign / fused_update_vstats / fast_gather.  All integer outputs
// (labels, counts, permutations) and the fixed-point query centroids are
// reproducible bit for bit: distances are fp32 fused-multiply-add chains in a
// fixed order, sums are either integers or accumulated in grouped row order by
// one owner warp.
#include <mutex>

#include "common.cuh"
#include "internal.h"

namespace t2t {

// ---------------------------------------------------------------------------
// assignment, all-exact form (the definition the tensor-core path must reproduce)
// ---------------------------------------------------------------------------
constexpr int AS_THREADS = 256;
constexpr int AS_RPT = 2;                       // rows per thread
constexpr int AS_ROWS = AS_THREADS * AS_RPT;    // rows per CTA
constexpr int AS_CT = 128;                      // centroids staged per step

__global__ void __launch_bounds__(AS_THREADS) assign_exact_kernel(const __nv_bfloat16* __restrict__ X,
                                                            const __nv_bfloat16* __restrict__ cen,
                                                            int* __restrict__ labels, int N, int Cn,
                                                            int pin_begin, int pin_label) {
  __shared__ __align__(16) float sC[AS_CT][kR];   // -2 c
  __shared__ float sN[AS_CT];                     // ||c||^2, +inf for padding
  const int h = blockIdx.y, tid = threadIdx.x;
  const __nv_bfloat16* Xh = X + (size_t)h * N * kR;
  const __nv_bfloat16* ch = cen + (size_t)h * Cn * kR;

  float x[AS_RPT][kR];
  int rows[AS_RPT];
#pragma unroll
  for (int u = 0; u < AS_RPT; ++u) {
    rows[u] = blockIdx.x * AS_ROWS + u * AS_THREADS + tid;
    const int r = rows[u] < N ? rows[u] : N - 1;
    const uint4* p = reinterpret_cast<const uint4*>(Xh + (size_t)r * kR);
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint4 w = p[g];
      x[u][8 * g + 0] = bf_lo(w.x); x[u][8 * g + 1] = bf_hi(w.x);
      x[u][8 * g + 2] = bf_lo(w.y); x[u][8 * g + 3] = bf_hi(w.y);
      x[u][8 * g + 4] = bf_lo(w.z); x[u][8 * g + 5] = bf_hi(w.z);
      x[u][8 * g + 6] = bf_lo(w.w); x[u][8 * g + 7] = bf_hi(w.w);
    }
  }
  float best[AS_RPT];
  int bidx[AS_RPT];
#pragma unroll
  for (int u = 0; u < AS_RPT; ++u) { best[u] = INFINITY; bidx[u] = 0; }

  for (int cbase = 0; cbase < Cn; cbase += AS_CT) {
    __syncthreads();
#pragma unroll
    for (int i = 0; i < AS_CT * kR / AS_THREADS / 2; ++i) {
      const int idx = tid + AS_THREADS * i;            // pair index
      const int c = idx >> 4, k2 = (idx & 15) * 2;
      uint32_t w = 0;
      if (cbase + c < Cn) w = *reinterpret_cast<const uint32_t*>(ch + (size_t)(cbase + c) * kR + k2);
      sC[c][k2] = -2.0f * bf_lo(w);
      sC[c][k2 + 1] = -2.0f * bf_hi(w);
    }
    __syncthreads();
    if (tid < AS_CT) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < kR; ++k) {
        const float v = -0.5f * sC[tid][k];
        s = fmaf(v, v, s);
      }
      sN[tid] = (cbase + tid < Cn) ? s : INFINITY;
    }
    __syncthreads();
#pragma unroll 4
    for (int c = 0; c < AS_CT; ++c) {
      float d[AS_RPT];
      const float cn = sN[c];
#pragma unroll
      for (int u = 0; u < AS_RPT; ++u) d[u] = cn;
#pragma unroll
      for (int g = 0; g < kR / 4; ++g) {
        const float4 cv = *reinterpret_cast<const float4*>(&sC[c][4 * g]);
#pragma unroll
        for (int u = 0; u < AS_RPT; ++u) {
          d[u] = fmaf(x[u][4 * g + 0], cv.x, d[u]);
          d[u] = fmaf(x[u][4 * g + 1], cv.y, d[u]);
          d[u] = fmaf(x[u][4 * g + 2], cv.z, d[u]);
          d[u] = fmaf(x[u][4 * g + 3], cv.w, d[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < AS_RPT; ++u) {
        const bool better = d[u] < best[u];     // strict: the first (lowest) index wins ties
        best[u] = better ? d[u] : best[u];
        bidx[u] = better ? cbase + c : bidx[u];
      }
    }
  }
#pragma unroll
  for (int u = 0; u < AS_RPT; ++u) {
    if (rows[u] < N) {
      int lab = bidx[u];
      if (pin_begin >= 0 && rows[u] >= pin_begin) lab = pin_label;
      labels[(size_t)h * N + rows[u]] = lab;
    }
  }
}

// ---------------------------------------------------------------------------
// stable grouping: per-chunk histograms -> offsets -> scatter
// ---------------------------------------------------------------------------
constexpr int GR_CHUNK = 1024;   // rows per warp
constexpr int GR_WARPS = 4;

__global__ void __launch_bounds__(GR_WARPS * 32) hist_kernel(const int* __restrict__ lab,
                                                             int* __restrict__ chist, int N, int Cn,
                                                             int nChunk) {
  extern __shared__ int sh[];
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * GR_WARPS + warp;
  int* hh = sh + warp * Cn;
  for (int i = lane; i < Cn; i += 32) hh[i] = 0;
  __syncwarp();
  if (chunk >= nChunk) return;
  const int* labh = lab + (size_t)h * N;
  const int r0 = chunk * GR_CHUNK, r1 = min(N, r0 + GR_CHUNK);
  for (int r = r0; r < r1; r += 32) {
    const int row = r + lane;
    int c = row < r1 ? labh[row] : -1;
    if ((unsigned)c >= (unsigned)Cn) c = -1;      // a label outside [0, Cn) is ignored, never indexed
    const unsigned peers = __match_any_sync(0xffffffffu, c);
    if (c >= 0 && lane == __ffs(peers) - 1) hh[c] += __popc(peers);
    __syncwarp();
  }
  int* out = chist + ((size_t)h * nChunk + chunk) * Cn;
  for (int i = lane; i < Cn; i += 32) out[i] = hh[i];
}

// One CTA per head: counts, exclusive cluster bases, and the write offset of
// every (chunk, cluster) pair, in place of the histogram.
__global__ void __launch_bounds__(1024) offsets_kernel(int* __restrict__ chist, int* __restrict__ counts,
                                                       int* __restrict__ cbase, int Cn, int nChunk) {
  __shared__ int wsum[32];
  __shared__ int carry_s;
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int* ch = chist + (size_t)h * nChunk * Cn;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < Cn; c0 += 1024) {
    const int c = c0 + tid;
    int tot = 0;
    if (c < Cn)
      for (int k = 0; k < nChunk; ++k) tot += ch[(size_t)k * Cn + c];
    int inc = warp_incl_scan(tot, lane);
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    if (warp == 0) {
      int w = wsum[lane];
      w = warp_incl_scan(w, lane);
      wsum[lane] = w;
    }
    __syncthreads();
    const int carry = carry_s;
    const int base = carry + inc - tot + (warp > 0 ? wsum[warp - 1] : 0);
    if (c < Cn) {
      counts[(size_t)h * Cn + c] = tot;
      cbase[(size_t)h * Cn + c] = base;
      int r = base;
      for (int k = 0; k < nChunk; ++k) {
        const int t = ch[(size_t)k * Cn + c];
        ch[(size_t)k * Cn + c] = r;
        r += t;
      }
    }
    __syncthreads();
    if (tid == 0) carry_s = carry + wsum[31];
    __syncthreads();
  }
}

__global__ void __launch_bounds__(GR_WARPS * 32) scatter_kernel(const int* __restrict__ lab,
                                                                const int* __restrict__ choff,
                                                                int* __restrict__ perm, int N, int Cn,
                                                                int nChunk) {
  extern __shared__ int sh[];
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x * GR_WARPS + warp;
  if (chunk >= nChunk) return;
  int* cur = sh + warp * Cn;
  const int* off = choff + ((size_t)h * nChunk + chunk) * Cn;
  for (int i = lane; i < Cn; i += 32) cur[i] = off[i];
  __syncwarp();
  const int* labh = lab + (size_t)h * N;
  int* out = perm + (size_t)h * N;
  const int r0 = chunk * GR_CHUNK, r1 = min(N, r0 + GR_CHUNK);
  for (int r = r0; r < r1; r += 32) {
    const int row = r + lane;
    int c = row < r1 ? labh[row] : -1;
    if ((unsigned)c >= (unsigned)Cn) c = -1;
    const unsigned peers = __match_any_sync(0xffffffffu, c);
    const int leader = __ffs(peers) - 1;
    const int rank = __popc(peers & ((1u << lane) - 1u));
    int base = 0;
    if (c >= 0 && lane == leader) {
      base = cur[c];
      cur[c] = base + __popc(peers);
    }
    base = __shfl_sync(0xffffffffu, base, leader);
    if (c >= 0) out[base + rank] = row;
    __syncwarp();
  }
}

static void launch_group(const int* lab, int* chist, int* counts, int* cbase, int* perm, int H, int N,
                         int Cn, cudaStream_t st) {
  const int nChunk = cdiv(N, GR_CHUNK);
  const size_t sh = (size_t)GR_WARPS * Cn * sizeof(int);
  hist_kernel<<<dim3(cdiv(nChunk, GR_WARPS), H), GR_WARPS * 32, sh, st>>>(lab, chist, N, Cn, nChunk);
  offsets_kernel<<<H, 1024, 0, st>>>(chist, counts, cbase, Cn, nChunk);
  scatter_kernel<<<dim3(cdiv(nChunk, GR_WARPS), H), GR_WARPS * 32, sh, st>>>(lab, chist, perm, N, Cn, nChunk);
}

// ---------------------------------------------------------------------------
// centroid updates (one owner warp per cluster, lane = dimension)
// ---------------------------------------------------------------------------
constexpr int CS_WARPS = 4;
constexpr int CS_UNR = 8;

// Exact integer sums of rint(x * 2^15); mean rounded once to bf16.
__global__ void __launch_bounds__(CS_WARPS * 32) fixed_mean_kernel(
    const __nv_bfloat16* __restrict__ X, const int* __restrict__ perm, const int* __restrict__ counts,
    const int* __restrict__ cbase, const __nv_bfloat16* __restrict__ old, __nv_bfloat16* __restrict__ newc,
    int N, int Cn) {
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * CS_WARPS + warp;
  if (c >= Cn) return;
  const int cnt = counts[(size_t)h * Cn + c];
  const int* srt = perm + (size_t)h * N + cbase[(size_t)h * Cn + c];
  const __nv_bfloat16* Xh = X + (size_t)h * N * kR;
  // Integer sums do not depend on the order: four lanes read one 64-byte row (16 bytes = 8 dimensions each),
  // so a load instruction covers eight rows; the eight row slots are added up by shuffles at the end.
  const int slot = lane >> 2, part = lane & 3;
  long long acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  constexpr int U = 4;
  for (int i = 0; i < cnt; i += 8 * U) {
    uint4 w[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int j = i + 8 * u + slot;
      w[u] = j < cnt ? *reinterpret_cast<const uint4*>(Xh + (size_t)srt[j] * kR + part * 8) : make_uint4(0u, 0u, 0u, 0u);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const uint32_t ws[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        acc[2 * e] += (long long)__float2int_rn(bf_lo(ws[e]) * 32768.0f);
        acc[2 * e + 1] += (long long)__float2int_rn(bf_hi(ws[e]) * 32768.0f);
      }
    }
  }
#pragma unroll
  for (int d = 4; d < 32; d <<= 1)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], d);
  if (slot == 0) {
    // lane `part` holds dimensions 8 part .. 8 part + 7
    const size_t o = ((size_t)h * Cn + c) * kR + part * 8;
    uint32_t outw[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      __nv_bfloat16 lo, hi;
      if (cnt) {
        lo = __float2bfloat16_rn((float)acc[2 * e] / (32768.0f * (float)cnt));
        hi = __float2bfloat16_rn((float)acc[2 * e + 1] / (32768.0f * (float)cnt));
      } else {
        lo = old[o + 2 * e];
        hi = old[o + 2 * e + 1];
      }
      outw[e] = (uint32_t)__bfloat16_as_ushort(lo) | ((uint32_t)__bfloat16_as_ushort(hi) << 16);
    }
    *reinterpret_cast<uint4*>(newc + o) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
  }
}

// Key side: fp32 sums accumulated one row at a time in grouped order, then the
// fp32 mean, its bf16 rounding and the scaled scoring centroid.
__global__ void __launch_bounds__(CS_WARPS * 32) key_mean_kernel(
    const __nv_bfloat16* __restrict__ X, const int* __restrict__ perm, const int* __restrict__ counts,
    const int* __restrict__ cbase, const __nv_bfloat16* __restrict__ old, float* __restrict__ ck2,
    __nv_bfloat16* __restrict__ ck16, __nv_bfloat16* __restrict__ cks16, float scale, int N, int Cn) {
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * CS_WARPS + warp;
  if (c >= Cn) return;
  const int cnt = counts[(size_t)h * Cn + c];
  const int* srt = perm + (size_t)h * N + cbase[(size_t)h * Cn + c];
  const __nv_bfloat16* Xh = X + (size_t)h * N * kR;
  float acc = 0.f;
  for (int i = 0; i < cnt; i += CS_UNR) {
    float v[CS_UNR];
#pragma unroll
    for (int u = 0; u < CS_UNR; ++u)
      v[u] = (i + u < cnt) ? bf_to_f(Xh[(size_t)srt[i + u] * kR + lane]) : 0.f;
#pragma unroll
    for (int u = 0; u < CS_UNR; ++u)
      if (i + u < cnt) acc += v[u];
  }
  const size_t o = ((size_t)h * Cn + c) * kR + lane;
  const float m = cnt ? acc / (float)cnt : bf_to_f(old[o]);
  ck2[o] = m;
  ck16[o] = __float2bfloat16_rn(m);
  cks16[o] = __float2bfloat16_rn(m * scale);
}

// V_sorted = V[perm] and fp32 value sums in grouped order; lane owns 4 dims.
__global__ void __launch_bounds__(CS_WARPS * 32) vgather_kernel(
    const __nv_bfloat16* __restrict__ V, const int* __restrict__ perm, const int* __restrict__ counts,
    const int* __restrict__ cbase, __nv_bfloat16* __restrict__ V_sorted, float* __restrict__ vsum, int N,
    int Cn, long long v_row_stride, long long v_head_stride) {
  const int h = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c = blockIdx.x * CS_WARPS + warp;
  if (c >= Cn) return;
  const int cnt = counts[(size_t)h * Cn + c];
  const int bs = cbase[(size_t)h * Cn + c];
  const int* srt = perm + (size_t)h * N + bs;
  const __nv_bfloat16* Vh = V + (size_t)h * v_head_stride;      // strides in elements: V may be a view of [N, H, 128]
  __nv_bfloat16* Vs = V_sorted + ((size_t)h * N + bs) * kD;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  for (int i = 0; i < cnt; i += CS_UNR) {
    uint2 w[CS_UNR];
#pragma unroll
    for (int u = 0; u < CS_UNR; ++u) {
      w[u] = make_uint2(0u, 0u);
      if (i + u < cnt) w[u] = __ldcs(reinterpret_cast<const uint2*>(Vh + (size_t)srt[i + u] * v_row_stride + lane * 4));
    }
#pragma unroll
    for (int u = 0; u < CS_UNR; ++u) {
      if (i + u < cnt) {
        *reinterpret_cast<uint2*>(Vs + (size_t)(i + u) * kD + lane * 4) = w[u];
        a0 += bf_lo(w[u].x); a1 += bf_hi(w[u].x);
        a2 += bf_lo(w[u].y); a3 += bf_hi(w[u].y);
      }
    }
  }
  *reinterpret_cast<float4*>(vsum + ((size_t)h * Cn + c) * kD + lane * 4) = make_float4(a0, a1, a2, a3);
}

constexpr int VM_BLOCKS = 32;
__global__ void __launch_bounds__(256) vmax_kernel(const float* __restrict__ vsum, float* __restrict__ bmax,
                                                   int Cn) {
  __shared__ float red[8];
  const int h = blockIdx.y;
  const size_t CE = (size_t)Cn * kD;
  float mx = 0.f;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < CE; i += (size_t)VM_BLOCKS * 256)
    mx = fmaxf(mx, fabsf(vsum[(size_t)h * CE + i]));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, red[i]);
    bmax[h * VM_BLOCKS + blockIdx.x] = mx;
  }
}

// lam = max(1, max|vsum| / 32768); sumv = bf16(vsum * (1 / lam)).
__global__ void __launch_bounds__(256) vscale_kernel(const float* __restrict__ vsum,
                                                     const float* __restrict__ bmax,
                                                     __nv_bfloat16* __restrict__ sumv, float* __restrict__ lam,
                                                     int Cn) {
  const int h = blockIdx.y;
  float mx = 0.f;
  for (int i = 0; i < VM_BLOCKS; ++i) mx = fmaxf(mx, bmax[h * VM_BLOCKS + i]);
  const float l = fmaxf(1.0f, mx / 32768.0f);
  if (blockIdx.x == 0 && threadIdx.x == 0) lam[h] = l;
  const float inv = 1.0f / l;
  const size_t CE = (size_t)Cn * kD;
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < CE; i += (size_t)gridDim.x * 256)
    sumv[(size_t)h * CE + i] = __float2bfloat16_rn(vsum[(size_t)h * CE + i] * inv);
}

static void launch_vstats(const __nv_bfloat16* V, const int* perm, const int* counts, const int* cbase,
                          __nv_bfloat16* V_sorted, __nv_bfloat16* sumv, float* lam, float* vsum,
                          float* bmax, int H, int N, int Cn, long long v_row_stride, long long v_head_stride,
                          cudaStream_t st) {
  vgather_kernel<<<dim3(cdiv(Cn, CS_WARPS), H), CS_WARPS * 32, 0, st>>>(V, perm, counts, cbase, V_sorted, vsum, N, Cn,
                                                                        v_row_stride, v_head_stride);
  vmax_kernel<<<dim3(VM_BLOCKS, H), 256, 0, st>>>(vsum, bmax, Cn);
  vscale_kernel<<<dim3(64, H), 256, 0, st>>>(vsum, bmax, sumv, lam, Cn);
}

// exclusive scan of counts per head (reuse calls hold counts but not bases)
__global__ void __launch_bounds__(1024) bases_kernel(const int* __restrict__ counts, int* __restrict__ cbase,
                                                     int Cn) {
  __shared__ int wsum[32];
  __shared__ int carry_s;
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) carry_s = 0;
  __syncthreads();
  for (int c0 = 0; c0 < Cn; c0 += 1024) {
    const int c = c0 + tid;
    const int v = c < Cn ? counts[(size_t)h * Cn + c] : 0;
    int inc = warp_incl_scan(v, lane);
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    if (warp == 0) wsum[lane] = warp_incl_scan(wsum[lane], lane);
    __syncthreads();
    const int carry = carry_s;
    if (c < Cn) cbase[(size_t)h * Cn + c] = carry + inc - v + (warp > 0 ? wsum[warp - 1] : 0);
    __syncthreads();
    if (tid == 0) carry_s = carry + wsum[31];
    __syncthreads();
  }
}

// out[h, i, :] = x[h, perm[h, i], :], one thread per 16-byte chunk.
__global__ void __launch_bounds__(256) gather_rows_kernel(const uint4* __restrict__ x,
                                                          const int* __restrict__ perm,
                                                          uint4* __restrict__ out, int N, size_t total,
                                                          long long x_row_stride16, long long x_head_stride16) {
  const size_t id = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (id >= total) return;
  const size_t row = id >> 4;
  const int ch = (int)(id & 15);
  const size_t h = row / N;
  const int src = perm[row];
  out[id] = __ldcs(x + h * x_head_stride16 + (size_t)src * x_row_stride16 + ch);      // strides in 16-byte units
}

// ---------------------------------------------------------------------------
// workspace layouts
// ---------------------------------------------------------------------------
struct Carver {
  char* base;
  size_t off = 0;
  explicit Carver(void* b) : base((char*)b) {}
  template <class T>
  T* take(size_t n) {
    T* p = base ? reinterpret_cast<T*>(base + off) : nullptr;
    off += (n * sizeof(T) + 255) & ~(size_t)255;
    return p;
  }
};

struct KmmWs {
  int *qlab1, *chist, *cbase_q, *cbase_k, *amb;
  int *chist_k, *amb_k;      // the key side runs next to the query side and needs scratch of its own
  __nv_bfloat16* cq1;
  float *vsum, *bmax;
  size_t total;
};
static KmmWs kmm_layout(int H, int N, int CQ, int C, void* base) {
  Carver cv(base);
  KmmWs w;
  const int nChunk = cdiv(N, GR_CHUNK);
  w.qlab1 = cv.take<int>((size_t)H * N);
  w.amb = cv.take<int>((size_t)H * N + 1);
  w.chist = cv.take<int>((size_t)H * nChunk * CQ);
  w.amb_k = cv.take<int>((size_t)H * N + 1);
  w.chist_k = cv.take<int>((size_t)H * nChunk * C);
  w.cbase_q = cv.take<int>((size_t)H * CQ);
  w.cbase_k = cv.take<int>((size_t)H * C);
  w.cq1 = cv.take<__nv_bfloat16>((size_t)H * CQ * kR);
  w.vsum = cv.take<float>((size_t)H * C * kD);
  w.bmax = cv.take<float>((size_t)H * VM_BLOCKS);
  w.total = cv.off;
  return w;
}

struct VstatWs {
  int* cbase;
  float *vsum, *bmax;
  size_t total;
};
static VstatWs vstat_layout(int H, int C, void* base) {
  Carver cv(base);
  VstatWs w;
  w.cbase = cv.take<int>((size_t)H * C);
  w.vsum = cv.take<float>((size_t)H * C * kD);
  w.bmax = cv.take<float>((size_t)H * VM_BLOCKS);
  w.total = cv.off;
  return w;
}

struct UpdWs {
  int *chist, *cbase, *perm;
  size_t total;
};
static UpdWs upd_layout(int H, int N, int Cn, void* base) {
  Carver cv(base);
  UpdWs w;
  w.chist = cv.take<int>((size_t)H * cdiv(N, GR_CHUNK) * Cn);
  w.cbase = cv.take<int>((size_t)H * Cn);
  w.perm = cv.take<int>((size_t)H * N);
  w.total = cv.off;
  return w;
}

static bool group_smem_ok(int Cn) {
  return (size_t)GR_WARPS * Cn * sizeof(int) <= 48 * 1024;
}

static int finish() { return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA; }

// A stream of the library's own per device, for work that is independent of what the caller's stream is doing
// inside one call: forked from the caller's stream by an event and joined back by another before the call
// returns, so the caller sees one ordered call.  The mutex is held while a call issues its work: two host
// threads must not interleave their records of the shared events.
struct SideStream {
  bool ready;
  cudaStream_t stream;
  cudaEvent_t fork, join;
  std::mutex issue;
};
static SideStream* side_stream() {
  static SideStream table[64];
  static std::mutex create;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(create);
  SideStream* s = &table[dev];
  if (!s->ready) {
    if (cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&s->fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s->join, cudaEventDisableTiming) != cudaSuccess)
      return nullptr;
    s->ready = true;
  }
  return s;
}

}  // namespace t2t

using namespace t2t;
typedef __nv_bfloat16 bf16;

extern "C" int t2t_version(void) { return 100; }

extern "C" int t2t_assign_exact(const void* x, const void* cen, void* labels, int H, int N, int Cn, int pin_begin,
                                int pin_label, cudaStream_t st) {
  if (!x || !cen || !labels || H <= 0 || N <= 0 || Cn <= 0) return T2T_ERR_ARG;
  assign_exact_kernel<<<dim3(cdiv(N, AS_ROWS), H), AS_THREADS, 0, st>>>((const bf16*)x, (const bf16*)cen,
                                                                        (int*)labels, N, Cn, pin_begin, pin_label);
  return finish();
}

extern "C" size_t t2t_assign_ws_bytes(int H, int N) { return assign_ws_bytes(H, N); }

extern "C" int t2t_assign(const void* x, const void* cen, void* labels, int H, int N, int Cn, int pin_begin,
                          int pin_label, void* ws, size_t ws_bytes, int* d_status, cudaStream_t st) {
  if (!x || !cen || !labels || !ws || H <= 0 || N <= 0 || Cn <= 0) return T2T_ERR_ARG;
  if (ws_bytes < assign_ws_bytes(H, N)) return T2T_ERR_WORKSPACE;
  return launch_assign((const bf16*)x, (const bf16*)cen, (int*)labels, H, N, Cn, pin_begin, pin_label, (int*)ws,
                       d_status, st);
}

extern "C" size_t t2t_centroid_update_ws_bytes(int H, int N, int Cn) { return upd_layout(H, N, Cn, nullptr).total; }

extern "C" int t2t_centroid_update(const void* x, const void* labels, const void* old, void* newc, void* counts,
                                   int H, int N, int Cn, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (!x || !labels || !old || !newc || !counts || !ws || H <= 0 || N <= 0 || Cn <= 0 || !group_smem_ok(Cn))
    return T2T_ERR_ARG;
  UpdWs w = upd_layout(H, N, Cn, ws);
  if (ws_bytes < w.total) return T2T_ERR_WORKSPACE;
  launch_group((const int*)labels, w.chist, (int*)counts, w.cbase, w.perm, H, N, Cn, st);
  fixed_mean_kernel<<<dim3(cdiv(Cn, CS_WARPS), H), CS_WARPS * 32, 0, st>>>(
      (const bf16*)x, w.perm, (const int*)counts, w.cbase, (const bf16*)old, (bf16*)newc, N, Cn);
  return finish();
}

extern "C" size_t t2t_kmeans_maintain_ws_bytes(int H, int N, int CQ, int C) {
  return kmm_layout(H, N, CQ, C, nullptr).total;
}

extern "C" int t2t_kmeans_maintain_strided(const void* QU, const void* KU, const void* V, long long v_row_stride, long long v_head_stride, const void* cq0,
                                   const void* ck0, void* qlab, void* cq2, void* klab, void* ck2, void* ck16,
                                   void* cks16, void* qcounts, void* qperm, void* kcounts, void* kperm,
                                   void* V_sorted, void* sumv, void* lam, float scale, int H, int N, int CQ,
                                   int C, int pin_tail, void* ws, size_t ws_bytes, int* d_status,
                                   cudaStream_t st) {
  if (v_row_stride < kD || v_head_stride <= 0 || (v_row_stride & 3) || (v_head_stride & 3)) return T2T_ERR_ARG;
  if (!QU || !KU || !V || !cq0 || !ck0 || !qlab || !cq2 || !klab || !ck2 || !ck16 || !cks16 || !qcounts ||
      !qperm || !kcounts || !kperm || !V_sorted || !sumv || !lam || !ws)
    return T2T_ERR_ARG;
  if (H <= 0 || N <= 0 || CQ <= 0 || C != kC || pin_tail < 0 || pin_tail > N || !group_smem_ok(CQ))
    return T2T_ERR_ARG;
  KmmWs w = kmm_layout(H, N, CQ, C, ws);
  if (ws_bytes < w.total) return T2T_ERR_WORKSPACE;
  int rc;
  const dim3 qgrid(cdiv(CQ, CS_WARPS), H), kgrid(cdiv(C, CS_WARPS), H);
  // The key side (assignment, grouping, means, value statistics) does not depend on the query side: it runs on
  // the library's side stream, next to the two query passes on the caller's.
  SideStream* side = side_stream();
  if (!side) return T2T_ERR_CUDA;
  std::lock_guard<std::mutex> issuing(side->issue);
  const cudaStream_t sk = side->stream;
  if (cudaEventRecord(side->fork, st) != cudaSuccess || cudaStreamWaitEvent(sk, side->fork, 0) != cudaSuccess)
    return T2T_ERR_CUDA;
  rc = launch_assign((const bf16*)KU, (const bf16*)ck0, (int*)klab, H, N, C, pin_tail > 0 ? N - pin_tail : -1,
                     C - 1, w.amb_k, d_status, sk);
  if (rc == T2T_OK) {
    launch_group((const int*)klab, w.chist_k, (int*)kcounts, w.cbase_k, (int*)kperm, H, N, C, sk);
    key_mean_kernel<<<kgrid, CS_WARPS * 32, 0, sk>>>((const bf16*)KU, (const int*)kperm, (const int*)kcounts,
                                                    w.cbase_k, (const bf16*)ck0, (float*)ck2, (bf16*)ck16,
                                                    (bf16*)cks16, scale, N, C);
    launch_vstats((const bf16*)V, (const int*)kperm, (const int*)kcounts, w.cbase_k, (bf16*)V_sorted, (bf16*)sumv,
                  (float*)lam, w.vsum, w.bmax, H, N, C, v_row_stride, v_head_stride, sk);
  }
  const bool recorded = cudaEventRecord(side->join, sk) == cudaSuccess;
  // whatever happens below, the caller's stream ends up ordered behind the side stream again
  auto join = [&]() { return recorded && cudaStreamWaitEvent(st, side->join, 0) == cudaSuccess; };
  if (rc != T2T_OK || !recorded) {
    join();
    return rc != T2T_OK ? rc : T2T_ERR_CUDA;
  }
  // queries, pass 1
  rc = launch_assign((const bf16*)QU, (const bf16*)cq0, w.qlab1, H, N, CQ, -1, 0, w.amb, d_status, st);
  if (rc != T2T_OK) { join(); return rc; }
  launch_group(w.qlab1, w.chist, (int*)qcounts, w.cbase_q, (int*)qperm, H, N, CQ, st);
  fixed_mean_kernel<<<qgrid, CS_WARPS * 32, 0, st>>>((const bf16*)QU, (const int*)qperm, (const int*)qcounts,
                                                    w.cbase_q, (const bf16*)cq0, w.cq1, N, CQ);
  // queries, pass 2
  rc = launch_assign((const bf16*)QU, w.cq1, (int*)qlab, H, N, CQ, -1, 0, w.amb, d_status, st);
  if (rc != T2T_OK) { join(); return rc; }
  launch_group((const int*)qlab, w.chist, (int*)qcounts, w.cbase_q, (int*)qperm, H, N, CQ, st);
  fixed_mean_kernel<<<qgrid, CS_WARPS * 32, 0, st>>>((const bf16*)QU, (const int*)qperm, (const int*)qcounts,
                                                    w.cbase_q, w.cq1, (bf16*)cq2, N, CQ);
  if (!join()) return T2T_ERR_CUDA;
  return finish();
}

extern "C" int t2t_kmeans_maintain(const void* QU, const void* KU, const void* V, const void* cq0,
                                   const void* ck0, void* qlab, void* cq2, void* klab, void* ck2, void* ck16,
                                   void* cks16, void* qcounts, void* qperm, void* kcounts, void* kperm,
                                   void* V_sorted, void* sumv, void* lam, float scale, int H, int N, int CQ,
                                   int C, int pin_tail, void* ws, size_t ws_bytes, int* d_status,
                                   cudaStream_t st) {
  return t2t_kmeans_maintain_strided(QU, KU, V, (long long)kD, (long long)N * kD, cq0, ck0, qlab, cq2, klab, ck2, ck16, cks16,
                                     qcounts, qperm, kcounts, kperm, V_sorted, sumv, lam, scale, H, N, CQ, C, pin_tail,
                                     ws, ws_bytes, d_status, st);
}

extern "C" size_t t2t_vstats_gather_ws_bytes(int H, int C) { return vstat_layout(H, C, nullptr).total; }

extern "C" int t2t_vstats_gather(const void* V, const void* kperm, const void* kcounts, void* V_sorted,
                                 void* sumv, void* lam, int H, int N, int C, void* ws, size_t ws_bytes,
                                 cudaStream_t st) {
  return t2t_vstats_gather_strided(V, (long long)kD, (long long)N * kD, kperm, kcounts, V_sorted, sumv, lam, H, N, C, ws,
                                   ws_bytes, st);
}

extern "C" int t2t_vstats_gather_strided(const void* V, long long v_row_stride, long long v_head_stride,
                                         const void* kperm, const void* kcounts, void* V_sorted, void* sumv, void* lam,
                                         int H, int N, int C, void* ws, size_t ws_bytes, cudaStream_t st) {
  if (!V || !kperm || !kcounts || !V_sorted || !sumv || !lam || !ws || H <= 0 || N <= 0 || C <= 0)
    return T2T_ERR_ARG;
  if (v_row_stride < kD || v_head_stride <= 0 || (v_row_stride & 3) || (v_head_stride & 3)) return T2T_ERR_ARG;
  VstatWs w = vstat_layout(H, C, ws);
  if (ws_bytes < w.total) return T2T_ERR_WORKSPACE;
  bases_kernel<<<H, 1024, 0, st>>>((const int*)kcounts, w.cbase, C);
  launch_vstats((const bf16*)V, (const int*)kperm, (const int*)kcounts, w.cbase, (bf16*)V_sorted, (bf16*)sumv,
                (float*)lam, w.vsum, w.bmax, H, N, C, v_row_stride, v_head_stride, st);
  return finish();
}

extern "C" int t2t_gather_rows(const void* x, const void* perm, void* out, int H, int N, cudaStream_t st) {
  return t2t_gather_rows_strided(x, (long long)kD, (long long)N * kD, perm, out, H, N, st);
}

extern "C" int t2t_gather_rows_strided(const void* x, long long x_row_stride, long long x_head_stride,
                                       const void* perm, void* out, int H, int N, cudaStream_t st) {
  if (!x || !perm || !out || H <= 0 || N <= 0) return T2T_ERR_ARG;
  if (x_row_stride < kD || x_head_stride <= 0 || (x_row_stride & 7) || (x_head_stride & 7)) return T2T_ERR_ARG;
  const size_t total = (size_t)H * N * 16;
  gather_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>((const uint4*)x, (const int*)perm,
                                                                     (uint4*)out, N, total, x_row_stride >> 3,
                                                                     x_head_stride >> 3);
  return finish();
}

// ---------------------------------------------------------------------------
// value statistics without any allocation
// ---------------------------------------------------------------------------
// Scratch for t2t_vstats_gather_static.  It is part of the library image: every
// GPU that loads the library holds these bytes until the process exits.
namespace t2t {
constexpr int kStaticMaxHeads = T2T_STATIC_VSTATS_MAX_HC / kC;
constexpr size_t kStaticScratchBytes =
    (((size_t)T2T_STATIC_VSTATS_MAX_HC * sizeof(int) + 255) & ~(size_t)255) +
    (((size_t)T2T_STATIC_VSTATS_MAX_HC * kD * sizeof(float) + 255) & ~(size_t)255) +
    (((size_t)kStaticMaxHeads * VM_BLOCKS * sizeof(float) + 255) & ~(size_t)255);
static __device__ __align__(256) unsigned char g_vstats_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
static void* g_vstats_scratch_addr[kMaxDevices];   // device address of the array, per device
}  // namespace t2t

extern "C" size_t t2t_vstats_gather_static_max_hc(void) { return T2T_STATIC_VSTATS_MAX_HC; }

extern "C" int t2t_vstats_gather_static(const void* V, const void* kperm, const void* kcounts, void* V_sorted,
                                        void* sumv, void* lam, int H, int N, int C, cudaStream_t st) {
  if (!V || !kperm || !kcounts || !V_sorted || !sumv || !lam || H <= 0 || N <= 0 || C <= 0) return T2T_ERR_ARG;
  // two limits: the per-cluster regions hold T2T_STATIC_VSTATS_MAX_HC clusters, the per-head one kStaticMaxHeads heads
  if (H > kStaticMaxHeads || (size_t)H * (size_t)C > (size_t)T2T_STATIC_VSTATS_MAX_HC) return T2T_ERR_TOO_LARGE;
  VstatWs probe = vstat_layout(H, C, nullptr);
  if (probe.total > kStaticScratchBytes) return T2T_ERR_TOO_LARGE;
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return T2T_ERR_CUDA;
  if (!g_vstats_scratch_addr[dev]) {
    // In host code the array's name is only a handle; the kernels need the
    // address it has on the current device.
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_vstats_scratch) != cudaSuccess || !p) return T2T_ERR_CUDA;
    g_vstats_scratch_addr[dev] = p;
  }
  VstatWs w = vstat_layout(H, C, g_vstats_scratch_addr[dev]);
  // Every word of the scratch that is read is written first in the same call
  // (bases, sums and block maxima cover all H * C clusters), so nothing has to
  // be cleared although the array keeps the previous call's contents.
  bases_kernel<<<H, 1024, 0, st>>>((const int*)kcounts, w.cbase, C);
  launch_vstats((const bf16*)V, (const int*)kperm, (const int*)kcounts, w.cbase, (bf16*)V_sorted, (bf16*)sumv,
                (float*)lam, w.vsum, w.bmax, H, N, C, (long long)kD, (long long)N * kD, st);
  return finish();
}
