// Fused scoring + budgeted cluster selection + query-cluster union.
//
// Replaces the reference's score matrix (torch.bmm into gl [H,N,2048],
// token2tile/operator/deploy_step.py:394) and its select_union extension
// (kernels/select_union/src/kernel.cu): the 2048 scores of a query live only
// in the registers of one warp.
//
// Per query row, one warp:
//   1. scores g_c = sum_k QU[k] * cks[c][k] as an fp32 fused-multiply-add
//      chain over k = 0..31 (64 clusters per lane), rounded to fp16 and mapped
//      to an order-preserving 16-bit key;
//   2. finds the largest key v* whose "clusters with key >= v*" hold at least
//      ns tokens, by a 16-step warp-level bitwise search (a radix select on the
//      key bits with size-weighted counts);
//   3. selects key > v*, and among key == v* the lowest cluster indices while
//      the running token count is still below ns;
//   4. ORs the selection into the warp's mask for the query cluster.
// A CTA walks several query clusters of one head so the 128 KB of centroids
// are staged into shared memory once.
#include "common.cuh"
#include "internal.h"

namespace t2t {

constexpr int SEL_WARPS = 16;
constexpr int SEL_THREADS = SEL_WARPS * 32;
constexpr int SEL_CK_WORDS = kR * (kC / 2);     // bf16 pairs, [k][pair]

__device__ __forceinline__ int key_from_score(float s) {
  // fp16 bit pattern, low 15 bits flipped for negatives, biased to 0..65535.
  unsigned u = __half_as_ushort(__float2half_rn(s));
  u ^= ((u >> 15) & 1u) * 0x7FFFu;
  return (int)((u ^ 0x8000u) & 0xFFFFu);
}

// Centroids of one head, transposed into [k][cluster pair] so that a lane reads
// the pair (2 lane + 64 j, 2 lane + 64 j + 1) of every j without bank conflicts.
__device__ __forceinline__ void stage_centroids(uint32_t* sCk, const __nv_bfloat16* __restrict__ ckh, int tid) {
  for (int idx = tid; idx < (kC / 2) * (kR / 2); idx += SEL_THREADS) {
    const int p = idx & (kC / 2 - 1), kk = (idx >> 10) * 2;
    const uint32_t w0 = *reinterpret_cast<const uint32_t*>(ckh + (size_t)(2 * p) * kR + kk);
    const uint32_t w1 = *reinterpret_cast<const uint32_t*>(ckh + (size_t)(2 * p + 1) * kR + kk);
    sCk[kk * (kC / 2) + p] = (w0 & 0xffffu) | (w1 << 16);
    sCk[(kk + 1) * (kC / 2) + p] = (w0 >> 16) | (w1 & 0xffff0000u);
  }
}

// Lane masks -> bitmap words: cluster 64 j + 2 lane + e is bit (2 lane + e) & 31 of
// word 2 j + (lane >= 16).  `emit(word, bits)` is called by lane 0.
template <class F>
__device__ __forceinline__ void masks_to_words(uint32_t selA, uint32_t selB, int lane, F emit) {
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const uint32_t two = ((j < 16 ? selA : selB) >> ((2 * j) & 31)) & 3u;
    const uint32_t contrib = two << (2 * (lane & 15));
    const uint32_t w0 = __reduce_or_sync(0xffffffffu, lane < 16 ? contrib : 0u);
    const uint32_t w1 = __reduce_or_sync(0xffffffffu, lane >= 16 ? contrib : 0u);
    if (lane == 0) {
      if (w0) emit(2 * j, w0);
      if (w1) emit(2 * j + 1, w1);
    }
  }
}

// The exact selection of one query row by one warp.  qv is QU[row][lane]; sCk the
// centroids as [k][cluster pair] bf16 pairs; lane owns clusters 64 j + 2 lane + e.
// Returns the lane's selection bits (bit (2 j + e) & 31 of gA for j < 16, of gB
// for j >= 16) and the selected token count rc.
__device__ __forceinline__ void select_row_exact(float qv, const uint32_t* __restrict__ sCk,
                                                 const int* __restrict__ sSize, int ns, int lane, uint32_t& gA_out,
                                                 uint32_t& gB_out, int& rc_out) {
  const int2* sSize2 = reinterpret_cast<const int2*>(sSize);
  float acc[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) acc[i] = 0.f;
#pragma unroll 2
  for (int k = 0; k < kR; ++k) {
    const float qk = __shfl_sync(0xffffffffu, qv, k);
    const uint32_t* ck = sCk + k * (kC / 2) + lane;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const uint32_t w = ck[j * 32];
      acc[2 * j] = fmaf(qk, bf_lo(w), acc[2 * j]);
      acc[2 * j + 1] = fmaf(qk, bf_hi(w), acc[2 * j + 1]);
    }
  }
  int kb[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) kb[i] = key_from_score(acc[i]);

  // largest v with  sum{ size_c : key_c >= v } >= ns
  int v = 0;
#pragma unroll 1
  for (int bit = 15; bit >= 0; --bit) {
    const int cand = v | (1 << bit);
    int s = 0;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const int2 sz = sSize2[j * 32 + lane];
      s += kb[2 * j] >= cand ? sz.x : 0;
      s += kb[2 * j + 1] >= cand ? sz.y : 0;
    }
    s = __reduce_add_sync(0xffffffffu, s);
    if (s >= ns) v = cand;
  }
  int sgt = 0, seq = 0, neq = 0;
  uint32_t gA = 0u, gB = 0u, eA = 0u, eB = 0u;
#pragma unroll
  for (int j = 0; j < 32; ++j) {
    const int2 sz = sSize2[j * 32 + lane];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int k16 = kb[2 * j + e];
      const int szc = e ? sz.y : sz.x;
      const uint32_t bitm = 1u << ((2 * j + e) & 31);
      if (k16 > v) { sgt += szc; if (j < 16) gA |= bitm; else gB |= bitm; }
      if (k16 == v) { seq += szc; ++neq; if (j < 16) eA |= bitm; else eB |= bitm; }
    }
  }
  sgt = __reduce_add_sync(0xffffffffu, sgt);
  seq = __reduce_add_sync(0xffffffffu, seq);
  neq = __reduce_add_sync(0xffffffffu, neq);
  int rc;
  if (neq == 1) {
    gA |= eA; gB |= eB;
    rc = sgt + seq;
  } else {
    // several clusters share the threshold key: take them by ascending
    // cluster index while fewer than ns tokens are selected
    const int R = ns - sgt;
    int run = 0;
    rc = sgt;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const uint32_t em = j < 16 ? eA : eB;
      unsigned b0 = __ballot_sync(0xffffffffu, (em >> ((2 * j) & 31)) & 1u);
      unsigned b1 = __ballot_sync(0xffffffffu, (em >> ((2 * j + 1) & 31)) & 1u);
      while (b0 | b1) {
        const int l = __ffs(b0 | b1) - 1;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const unsigned be = e ? b1 : b0;
          if ((be >> l) & 1u) {
            const int szc = sSize[64 * j + 2 * l + e];
            if (run < R) {
              if (lane == l) { if (j < 16) gA |= 1u << ((2 * j + e) & 31); else gB |= 1u << ((2 * j + e) & 31); }
              if (run + szc >= R) rc = sgt + run + szc;
            }
            run += szc;
          }
        }
        b0 &= ~(1u << l);
        b1 &= ~(1u << l);
      }
    }
  }
  gA_out = gA;
  gB_out = gB;
  rc_out = rc;
}

__global__ void __launch_bounds__(SEL_THREADS, 1) select_exact_kernel(
    const __nv_bfloat16* __restrict__ QU, const __nv_bfloat16* __restrict__ cks,
    const int* __restrict__ kcounts, const int* __restrict__ qperm, const int* __restrict__ tile_sizes,
    const int* __restrict__ ns_ptr, int* __restrict__ unip, int* __restrict__ rowcnt, int N, int CQ,
    int pin_tail) {
  extern __shared__ __align__(16) uint32_t smem_sel[];
  uint32_t* sCk = smem_sel;                                    // [32][1024]
  int* sSize = reinterpret_cast<int*>(sCk + SEL_CK_WORDS);     // [2048]
  uint32_t* sUnion = reinterpret_cast<uint32_t*>(sSize + kC);  // [64]
  int* sScan = reinterpret_cast<int*>(sUnion + 64);            // [32]
  int* sOff = sScan + 32;                                      // [CQ + 1]

  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __nv_bfloat16* ckh = cks + (size_t)h * kC * kR;

  stage_centroids(sCk, ckh, tid);
  for (int c = tid; c < kC; c += SEL_THREADS) sSize[c] = kcounts[(size_t)h * kC + c];
  // exclusive scan of the query-cluster sizes
  {
    int carry = 0;
    for (int c0 = 0; c0 < CQ; c0 += SEL_THREADS) {
      const int c = c0 + tid;
      const int v = c < CQ ? tile_sizes[(size_t)h * CQ + c] : 0;
      int inc = warp_incl_scan(v, lane);
      if (lane == 31) sScan[warp] = inc;
      __syncthreads();
      if (warp == 0) {
        const int w = lane < SEL_WARPS ? sScan[lane] : 0;
        sScan[lane] = warp_incl_scan(w, lane);
      }
      __syncthreads();
      if (c < CQ) sOff[c] = carry + inc - v + (warp > 0 ? sScan[warp - 1] : 0);
      carry += sScan[SEL_WARPS - 1];
      __syncthreads();
    }
    if (tid == 0) sOff[CQ] = carry;
  }
  __syncthreads();

  const int ns = *ns_ptr;
  for (int t = blockIdx.x; t < CQ; t += gridDim.x) {
    if (tid < 64) sUnion[tid] = 0u;
    __syncthreads();
    const int off = sOff[t];
    const int nrows = sOff[t + 1] - off;
    uint32_t selA = 0u, selB = 0u;     // bit 2 j' + e of cluster 64 j + 2 lane + e; A: j < 16, B: j >= 16

    for (int rr = warp; rr < nrows; rr += SEL_WARPS) {
      const int row = qperm[(size_t)h * N + off + rr];
      const float qv = bf_to_f(QU[((size_t)h * N + row) * kR + lane]);
      uint32_t gA, gB;
      int rc;
      select_row_exact(qv, sCk, sSize, ns, lane, gA, gB, rc);
      selA |= gA;
      selB |= gB;
      if (lane == 0) rowcnt[(size_t)h * N + row] = rc;
    }

    masks_to_words(selA, selB, lane, [&](int w, uint32_t bits) { atomicOr(&sUnion[w], bits); });
    __syncthreads();
    if (tid < 64) {
      uint32_t w = sUnion[tid];
      if (pin_tail > 0 && tid == 63) w |= 0x80000000u;
      unip[((size_t)h * CQ + t) * 64 + tid] = (int)w;
    }
    __syncthreads();
  }
}

// Rows the tensor-core kernel could not settle (select_tc.cu) are re-done here by
// the exact warp-per-row routine.  fixq holds, per head, a count followed by
// (row, query cluster) pairs.  Bits are OR-ed into the bitmap the fast kernel
// already wrote.
__global__ void __launch_bounds__(SEL_THREADS, 1) select_fix_kernel(
    const __nv_bfloat16* __restrict__ QU, const __nv_bfloat16* __restrict__ cks,
    const int* __restrict__ kcounts, const int* __restrict__ ns_ptr, int* __restrict__ unip,
    int* __restrict__ rowcnt, int N, int CQ, const int* __restrict__ fixq) {
  extern __shared__ __align__(16) uint32_t smem_sel[];
  uint32_t* sCk = smem_sel;
  int* sSize = reinterpret_cast<int*>(sCk + SEL_CK_WORDS);
  const int h = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int* q = fixq + (size_t)h * (2 * (size_t)N + 1);
  const int count = q[0];
  if (blockIdx.x * SEL_WARPS >= count) return;
  stage_centroids(sCk, cks + (size_t)h * kC * kR, tid);
  for (int c = tid; c < kC; c += SEL_THREADS) sSize[c] = kcounts[(size_t)h * kC + c];
  __syncthreads();
  const int ns = *ns_ptr;
  for (int e = blockIdx.x * SEL_WARPS + warp; e < count; e += gridDim.x * SEL_WARPS) {
    const int row = q[1 + 2 * e], t = q[2 + 2 * e] & 0xFFFFFF;      // top byte: why the fast kernel queued it
    const float qv = bf_to_f(QU[((size_t)h * N + row) * kR + lane]);
    uint32_t gA, gB;
    int rc;
    select_row_exact(qv, sCk, sSize, ns, lane, gA, gB, rc);
    if (lane == 0) rowcnt[(size_t)h * N + row] = rc;
    int* dst = unip + ((size_t)h * CQ + t) * 64;
    masks_to_words(gA, gB, lane, [&](int w, uint32_t bits) { atomicOr(reinterpret_cast<unsigned*>(dst) + w, bits); });
  }
}

size_t select_exact_smem(int CQ) { return (size_t)SEL_CK_WORDS * 4 + kC * 4 + 64 * 4 + 32 * 4 + (size_t)(CQ + 1) * 4; }

int launch_select_fix(const __nv_bfloat16* QU, const __nv_bfloat16* cks, const int* kcounts, const int* ns,
                      int* unip, int* rowcnt, int H, int N, int CQ, const int* fixq, cudaStream_t st) {
  const size_t smem = (size_t)SEL_CK_WORDS * 4 + kC * 4;
  if (cudaFuncSetAttribute(select_fix_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return T2T_ERR_CUDA;
  select_fix_kernel<<<dim3(8, H), SEL_THREADS, smem, st>>>(QU, cks, kcounts, ns, unip, rowcnt, N, CQ, fixq);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}

}  // namespace t2t

extern "C" int t2t_score_select_union_exact(const void* QU, const void* cks, const void* kcounts, const void* qperm,
                                      const void* tile_sizes, const int* ns, void* unip, void* rowcnt, int H,
                                      int N, int CQ, int pin_tail, cudaStream_t st) {
  using namespace t2t;
  if (!QU || !cks || !kcounts || !qperm || !tile_sizes || !ns || !unip || !rowcnt) return T2T_ERR_ARG;
  if (H <= 0 || N <= 0 || CQ <= 0 || N >= (1 << 24)) return T2T_ERR_ARG;
  const size_t smem = (size_t)SEL_CK_WORDS * 4 + kC * 4 + 64 * 4 + 32 * 4 + (size_t)(CQ + 1) * 4;
  if (smem > 227 * 1024) return T2T_ERR_ARG;
  if (cudaFuncSetAttribute(select_exact_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
    return T2T_ERR_CUDA;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int per_head = cdiv(10 * sms, H);
  if (per_head > CQ) per_head = CQ;
  select_exact_kernel<<<dim3(per_head, H), SEL_THREADS, smem, st>>>(
      (const __nv_bfloat16*)QU, (const __nv_bfloat16*)cks, (const int*)kcounts, (const int*)qperm,
      (const int*)tile_sizes, ns, (int*)unip, (int*)rowcnt, N, CQ, pin_tail);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}
