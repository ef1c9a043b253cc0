// Nearest-centroid assignment on the tensor cores with exact verification.
//
// The label of a row is DEFINED by the fp32 fused-multiply-add chain of
// assign_exact_kernel (kmeans.cu): d(i,c) = fma chain over k from ||c||^2 with
// x_k * (-2 c_k), lowest index on ties.  Evaluating that chain for every
// (row, centroid) pair costs N * C * 32 FMAs on the CUDA cores.  Here a tcgen05
// MMA (128 rows x 128 centroids x 32) produces approximate dot products, every
// thread keeps the best two distances of its row, and the tensor-core result is
// trusted only when the runner-up is further away than twice a bound on
// |approximate - chain|.  The few remaining rows are queued and re-evaluated
// with the exact chain over all centroids, so the labels are bit-identical to
// the all-exact kernel.
//
// Error bound.  With s~ the tensor-core sum and s the real sum of x_k c_k,
// |s~ - s| <= kappa * ||x|| ||c|| with kappa = 2^-16 (the measured error of the
// fp32 accumulation is below 2^-20; tests/test_gpu_stages.py checks it), the
// final fma adds 2^-24 |d~|, and the 32-step chain itself is within
// 2^-19 (||c||^2 + 2 ||x|| ||c||) of the real value.  All of it is covered by
//     eps_i = 2^-14 ||x_i|| max_c ||c|| + 2^-17 max_c ||c||^2 .
#include "common.cuh"
#include "internal.h"

namespace t2t {

constexpr int TA_ROWS = 128;
constexpr int TA_CH = 128;                     // centroids per chunk
constexpr int TA_SA = TA_ROWS * 128;           // 16 KB: rows padded to 128 B
constexpr int TA_SB = TA_CH * 128;             // 16 KB per stage
constexpr int TA_SMEM = TA_SA + 2 * TA_SB + 2 * TA_CH * 4 + 64 + 1024;

struct Top2 {
  float b1, b2;
  int i1;
};
__device__ __forceinline__ void top2_push(Top2& t, float d, int c) {
  const bool better = d < t.b1;                // strict: the first (lowest) index keeps a tie
  t.b2 = fminf(t.b2, fmaxf(d, t.b1));
  t.i1 = better ? c : t.i1;
  t.b1 = fminf(t.b1, d);
}

__global__ void __launch_bounds__(128, 4) assign_tc_kernel(const __nv_bfloat16* __restrict__ X,
                                                           const __nv_bfloat16* __restrict__ cen,
                                                           int* __restrict__ labels, int N, int Cn, int pin_begin,
                                                           int pin_label, int* __restrict__ amb,
                                                           int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base, sB = base + TA_SA;
  float* sCn = reinterpret_cast<float*>(sm + TA_SA + 2 * TA_SB);           // [2][TA_CH]
  uint64_t* bar = reinterpret_cast<uint64_t*>(sm + TA_SA + 2 * TA_SB + 2 * TA_CH * 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bar + 2);
  int* sCnMax = reinterpret_cast<int*>(bar + 3);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int h = blockIdx.y, row0 = blockIdx.x * TA_ROWS;
  const __nv_bfloat16* Xh = X + (size_t)h * N * kR;
  const __nv_bfloat16* ch = cen + (size_t)h * Cn * kR;

  if (warp == 0) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  if (tid == 0) {
    *abort_flag = 0;
    *sCnMax = 0;
    mbar_init(bar, 1);
    mbar_init_fence();
  }
  const int lch = tid & 3, lr0 = tid >> 2;     // 4 chunks of 16 B per 64-byte row
  auto load_rows = [&](uint32_t dst, const __nv_bfloat16* src, int first, int limit) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int r = lr0 + 32 * u;
      const bool valid = first + r < limit;
      cp_async16(dst + sw128(r, lch), src + (size_t)(valid ? first + r : 0) * kR + lch * 8, valid ? 16u : 0u);
    }
    cp_async_commit();
  };
  load_rows(sA, Xh, row0, N);
  load_rows(sB, ch, 0, Cn);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_lane = tmem_addr(tmem, warp * 32, 0);
  constexpr uint32_t idesc = make_idesc_bf16(128, TA_CH, false, false);

  Top2 ta{INFINITY, INFINITY, 0}, tb{INFINITY, INFINITY, 0};
  uint32_t ph = 0;
  bool dead = false;
  const int nch = cdiv(Cn, TA_CH);
  for (int j = 0; j < nch; ++j) {
    const int st = j & 1;
    if (j + 1 < nch) load_rows(sB + ((j + 1) & 1) * TA_SB, ch, (j + 1) * TA_CH, Cn);
    if (j + 1 < nch) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();                              // chunk j (and the row tile) is in shared memory
    {
      // ||c||^2 of centroid `tid` of this chunk, by the defining chain
      const uint8_t* rowp = sm + TA_SA + st * TA_SB;
      float s = 0.f;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint4 w = *reinterpret_cast<const uint4*>(rowp + sw128(tid, q4));
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float lo = bf_lo(ws[e]), hi = bf_hi(ws[e]);
          s = fmaf(lo, lo, s);
          s = fmaf(hi, hi, s);
        }
      }
      const bool real = j * TA_CH + tid < Cn;
      sCn[st * TA_CH + tid] = real ? s : INFINITY;
      if (real) atomicMax(sCnMax, __float_as_int(s));
    }
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int s2 = 0; s2 < 2; ++s2)
        umma_ss(tmem, make_sdesc(sA + s2 * 32, 16, 1024), make_sdesc(sB + st * TA_SB + s2 * 32, 16, 1024), idesc,
                s2 > 0 ? 1u : 0u);
      umma_commit(bar);
    }
    if (!mbar_wait(bar, ph, abort_flag)) { dead = true; break; }
    ph ^= 1u;
    tc_fence_after();
    const float* cn = sCn + st * TA_CH;
    const int cbase = j * TA_CH;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t v[32];
      tmem_ld32(t_lane + q * 32, v);
      tmem_wait_ld();
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float4 c4 = *reinterpret_cast<const float4*>(cn + q * 32 + g * 4);
        const int c = cbase + q * 32 + g * 4;
        top2_push(ta, fmaf(-2.0f, __uint_as_float(v[4 * g + 0]), c4.x), c);
        top2_push(tb, fmaf(-2.0f, __uint_as_float(v[4 * g + 1]), c4.y), c + 1);
        top2_push(ta, fmaf(-2.0f, __uint_as_float(v[4 * g + 2]), c4.z), c + 2);
        top2_push(tb, fmaf(-2.0f, __uint_as_float(v[4 * g + 3]), c4.w), c + 3);
      }
    }
    tc_fence_before();
    // the next iteration's first __syncthreads orders these TMEM reads before the next MMA
  }
  if (!dead) {
    // ||x||^2 of this thread's row
    float xn = 0.f;
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const uint4 w = *reinterpret_cast<const uint4*>(sm + sw128(tid, q4));
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float lo = bf_lo(ws[e]), hi = bf_hi(ws[e]);
        xn = fmaf(lo, lo, xn);
        xn = fmaf(hi, hi, xn);
      }
    }
    const float cnmax = __int_as_float(*sCnMax);
    const float eps = 6.103515625e-05f * sqrtf(xn) * sqrtf(cnmax) + 7.62939453125e-06f * cnmax;
    // merge the two column streams: smaller distance, lower index on equality
    const bool a_first = ta.b1 < tb.b1 || (ta.b1 == tb.b1 && ta.i1 < tb.i1);
    const float best = a_first ? ta.b1 : tb.b1;
    const int bi = a_first ? ta.i1 : tb.i1;
    const float second = fminf(fminf(ta.b2, tb.b2), a_first ? tb.b1 : ta.b1);
    const int row = row0 + tid;
    if (row < N) {
      const bool pinned = pin_begin >= 0 && row >= pin_begin;
      labels[(size_t)h * N + row] = pinned ? pin_label : bi;
      const bool sure = (second - best) > 2.0f * eps;      // false for NaN as well
      if (!sure && !pinned) {
        const int slot = atomicAdd(amb, 1);
        amb[1 + slot] = h * N + row;
      }
    }
  } else if (tid == 0 && status) {
    atomicExch(status, ST_WAIT_TIMEOUT);
  }
  cp_async_wait<0>();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

// Exact chain over all centroids for the queued rows; one warp per row.
__global__ void __launch_bounds__(256) assign_fix_kernel(const __nv_bfloat16* __restrict__ X,
                                                         const __nv_bfloat16* __restrict__ cen,
                                                         int* __restrict__ labels, int N, int Cn,
                                                         const int* __restrict__ amb) {
  const int lane = threadIdx.x & 31;
  const int warps = gridDim.x * (blockDim.x >> 5);
  const int count = amb[0];
  for (int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); e < count; e += warps) {
    const int gr = amb[1 + e];
    const int h = gr / N;
    const uint4* xp = reinterpret_cast<const uint4*>(X + (size_t)gr * kR);
    float x[kR];
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint4 w = xp[g];
      x[8 * g + 0] = bf_lo(w.x); x[8 * g + 1] = bf_hi(w.x);
      x[8 * g + 2] = bf_lo(w.y); x[8 * g + 3] = bf_hi(w.y);
      x[8 * g + 4] = bf_lo(w.z); x[8 * g + 5] = bf_hi(w.z);
      x[8 * g + 6] = bf_lo(w.w); x[8 * g + 7] = bf_hi(w.w);
    }
    float best = INFINITY;
    int bi = 0x7fffffff;
    for (int c = lane; c < Cn; c += 32) {
      const uint4* cp = reinterpret_cast<const uint4*>(cen + ((size_t)h * Cn + c) * kR);
      float cv[kR];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const uint4 w = cp[g];
        cv[8 * g + 0] = bf_lo(w.x); cv[8 * g + 1] = bf_hi(w.x);
        cv[8 * g + 2] = bf_lo(w.y); cv[8 * g + 3] = bf_hi(w.y);
        cv[8 * g + 4] = bf_lo(w.z); cv[8 * g + 5] = bf_hi(w.z);
        cv[8 * g + 6] = bf_lo(w.w); cv[8 * g + 7] = bf_hi(w.w);
      }
      float d = 0.f;
#pragma unroll
      for (int k = 0; k < kR; ++k) d = fmaf(cv[k], cv[k], d);
#pragma unroll
      for (int k = 0; k < kR; ++k) d = fmaf(x[k], -2.0f * cv[k], d);
      if (d < best) { best = d; bi = c; }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, m);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, m);
      if (ob < best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) labels[gr] = bi == 0x7fffffff ? 0 : bi;
  }
}

size_t assign_ws_bytes(int H, int N) { return ((size_t)H * N + 1) * sizeof(int); }

int launch_assign(const __nv_bfloat16* X, const __nv_bfloat16* cen, int* labels, int H, int N, int Cn,
                  int pin_begin, int pin_label, int* amb, int* d_status, cudaStream_t st) {
  if (cudaMemsetAsync(amb, 0, sizeof(int), st) != cudaSuccess) return T2T_ERR_CUDA;
  if (cudaFuncSetAttribute(assign_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TA_SMEM) != cudaSuccess)
    return T2T_ERR_CUDA;
  assign_tc_kernel<<<dim3(cdiv(N, TA_ROWS), H), 128, TA_SMEM, st>>>(X, cen, labels, N, Cn, pin_begin, pin_label,
                                                                    amb, d_status);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  assign_fix_kernel<<<2 * sms, 256, 0, st>>>(X, cen, labels, N, Cn, amb);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}

}  // namespace t2t
