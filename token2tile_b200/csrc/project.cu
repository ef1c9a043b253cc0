// Rank-32 projection  out[h, n, :] = bf16( x[h, n, :] . U[h] )  and the tensor
// core self-test.
//
// Replaces the two cuBLAS `torch.bmm` calls of the reference operator
// (token2tile/operator/deploy_step.py:321-324).  One CTA projects one tile of
// 128 rows with a single 128 x 32 x 128 tcgen05 MMA chain (fp32 accumulator in
// TMEM); several CTAs are resident per SM so that the loads of one overlap the
// epilogue of another.  The kernel is HBM-bound: it reads 256 B and writes
// 64 B per row.
#include "common.cuh"
#include "t2t_b200.h"

namespace t2t {

constexpr int PJ_ROWS = 128;
constexpr int PJ_SMEM_A = PJ_ROWS * kD * 2;        // 32 KB: two 64-column blocks of 16 KB
constexpr int PJ_SMEM_B = kR * kD * 2;             // 8 KB: two 64-column blocks of 4 KB
constexpr int PJ_SMEM = PJ_SMEM_A + PJ_SMEM_B + 64 + 1024;

__global__ void __launch_bounds__(128) project_kernel(const __nv_bfloat16* __restrict__ X,
                                                      const __nv_bfloat16* __restrict__ U,
                                                      __nv_bfloat16* __restrict__ out, int N,
                                                      long long x_row_stride, long long x_head_stride,
                                                      int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base, sB = base + PJ_SMEM_A;
  uint64_t* bar = reinterpret_cast<uint64_t*>(sm + PJ_SMEM_A + PJ_SMEM_B);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + PJ_SMEM_A + PJ_SMEM_B + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + PJ_SMEM_A + PJ_SMEM_B + 32);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int h = blockIdx.y;
  const int row0 = blockIdx.x * PJ_ROWS;

  if (warp == 0) {
    tmem_alloc(tmem_slot, 32);
    tmem_relinquish();
  }
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar, 1);
    mbar_init_fence();
  }

  // x tile: 128 rows x 16 chunks of 16 B, 16 consecutive threads per row.
  const __nv_bfloat16* Xh = X + (size_t)h * x_head_stride;      // strides in elements: x may be a view of [N, H, 128]
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int id = tid + 128 * i;
    const int row = id >> 4, ch = id & 15;
    const bool valid = row0 + row < N;
    const __nv_bfloat16* src = valid ? Xh + (size_t)(row0 + row) * x_row_stride + ch * 8 : Xh;
    cp_async16(sA + (ch >> 3) * (PJ_ROWS * 128) + sw128(row, ch & 7), src, valid ? 16u : 0u);
  }
  cp_async_commit();

  // U[h] is [128 d][32 j]; the B operand wants rows j with d contiguous.
  {
    const int d = tid;
    const uint4* up = reinterpret_cast<const uint4*>(U + ((size_t)h * kD + d) * kR);
    const uint32_t rowbase = (d >> 6) * (kR * 128) + ((d & 7) << 1);
    const uint32_t chunk = (d & 63) >> 3;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
      const uint4 w = up[g];
      const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int j = g * 8 + e * 2;
        *reinterpret_cast<unsigned short*>(sm + PJ_SMEM_A + rowbase + sw128(j, chunk)) =
            (unsigned short)(ws[e] & 0xffffu);
        *reinterpret_cast<unsigned short*>(sm + PJ_SMEM_A + rowbase + sw128(j + 1, chunk)) =
            (unsigned short)(ws[e] >> 16);
      }
    }
  }
  cp_async_wait<0>();
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (tid == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(128, kR, false, false);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const uint64_t ad = make_sdesc(sA + (s >> 2) * (PJ_ROWS * 128) + (s & 3) * 32, 16, 1024);
      const uint64_t bd = make_sdesc(sB + (s >> 2) * (kR * 128) + (s & 3) * 32, 16, 1024);
      umma_ss(tmem, ad, bd, idesc, s > 0 ? 1u : 0u);
    }
    umma_commit(bar);
  }
  const bool ok = mbar_wait(bar, 0, abort_flag);
  tc_fence_after();
  if (ok) {
    uint32_t v[32];
    tmem_ld32(tmem_addr(tmem, warp * 32, 0), v);
    tmem_wait_ld();
    const int row = row0 + tid;
    if (row < N) {
      uint4* dst = reinterpret_cast<uint4*>(out + ((size_t)h * N + row) * kR);
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 o;
        o.x = pack_bf2(__uint_as_float(v[8 * g + 0]), __uint_as_float(v[8 * g + 1]));
        o.y = pack_bf2(__uint_as_float(v[8 * g + 2]), __uint_as_float(v[8 * g + 3]));
        o.z = pack_bf2(__uint_as_float(v[8 * g + 4]), __uint_as_float(v[8 * g + 5]));
        o.w = pack_bf2(__uint_as_float(v[8 * g + 6]), __uint_as_float(v[8 * g + 7]));
        dst[g] = o;
      }
    }
  } else if (tid == 0 && status) {
    atomicExch(status, ST_WAIT_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 32);
}

// ---------------------------------------------------------------------------
// Tensor-core self-test: S = A . B^T (both operands K-major in shared memory),
// P = bf16(S / 16) written back over S in TMEM, O = P . V with P read from
// TMEM and V MN-major in shared memory.  These are exactly the operand forms
// the attention kernels use.
// ---------------------------------------------------------------------------
constexpr int ST_TILE = 128 * 128 * 2;   // 32 KB per operand
constexpr int ST_SMEM = 3 * ST_TILE + 64 + 1024;

__global__ void __launch_bounds__(128) umma_selftest_kernel(const __nv_bfloat16* __restrict__ A,
                                                            const __nv_bfloat16* __restrict__ B,
                                                            const __nv_bfloat16* __restrict__ V,
                                                            float* __restrict__ S_out,
                                                            float* __restrict__ O_out,
                                                            int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sA = base, sB = base + ST_TILE, sV = base + 2 * ST_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + 3 * ST_TILE);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + 3 * ST_TILE + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + 3 * ST_TILE + 32);
  const int tid = threadIdx.x, warp = tid >> 5;

  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bars + 0, 1);
    mbar_init(bars + 1, 1);
    mbar_init_fence();
  }
  const __nv_bfloat16* srcs[3] = {A, B, V};
  const uint32_t dsts[3] = {sA, sB, sV};
#pragma unroll
  for (int m = 0; m < 3; ++m) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int id = tid + 128 * i;
      const int row = id >> 4, ch = id & 15;
      cp_async16(dsts[m] + (ch >> 3) * 16384 + sw128(row, ch & 7), srcs[m] + row * 128 + ch * 8, 16u);
    }
  }
  cp_async_commit();
  cp_async_wait<0>();
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;

  if (tid == 0) {
    constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, false);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const uint64_t ad = make_sdesc(sA + (s >> 2) * 16384 + (s & 3) * 32, 16, 1024);
      const uint64_t bd = make_sdesc(sB + (s >> 2) * 16384 + (s & 3) * 32, 16, 1024);
      umma_ss(tS, ad, bd, idesc, s > 0 ? 1u : 0u);
    }
    umma_commit(bars + 0);
  }
  bool ok = mbar_wait(bars + 0, 0, abort_flag);
  tc_fence_after();
  if (ok) {
    uint32_t p[64];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tS, warp * 32, c * 32), v);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) S_out[tid * 128 + c * 32 + j] = __uint_as_float(v[j]);
#pragma unroll
      for (int j = 0; j < 16; ++j)
        p[c * 16 + j] = pack_bf2(__uint_as_float(v[2 * j]) * 0.0625f, __uint_as_float(v[2 * j + 1]) * 0.0625f);
    }
    uint32_t lo[32], hi[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) { lo[j] = p[j]; hi[j] = p[32 + j]; }
    tmem_st32(tmem_addr(tS, warp * 32, 0), lo);
    tmem_st32(tmem_addr(tS, warp * 32, 32), hi);
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (tid == 0 && !*abort_flag) {
    constexpr uint32_t idesc = make_idesc_bf16(128, 128, false, true);
#pragma unroll
    for (int s = 0; s < 8; ++s) {
      const uint64_t bd = make_sdesc(sV + s * 2048, 16384, 1024);
      umma_ts(tO, tS + s * 8, bd, idesc, s > 0 ? 1u : 0u);
    }
    umma_commit(bars + 1);
  }
  ok = ok && mbar_wait(bars + 1, 0, abort_flag);
  tc_fence_after();
  if (ok) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tO, warp * 32, c * 32), v);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 32; ++j) O_out[tid * 128 + c * 32 + j] = __uint_as_float(v[j]);
    }
  } else if (tid == 0 && status) {
    atomicExch(status, ST_WAIT_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace t2t

extern "C" int t2t_project(const void* x, const void* U, void* out, int H, int N, int* d_status,
                           cudaStream_t stream) {
  return t2t_project_strided(x, (long long)t2t::kD, (long long)N * t2t::kD, U, out, H, N, d_status, stream);
}

extern "C" int t2t_project_strided(const void* x, long long x_row_stride, long long x_head_stride, const void* U,
                                   void* out, int H, int N, int* d_status, cudaStream_t stream) {
  using namespace t2t;
  if (!x || !U || !out || H <= 0 || N <= 0) return T2T_ERR_ARG;
  if (x_row_stride < kD || x_head_stride <= 0 || (x_row_stride & 7) || (x_head_stride & 7)) return T2T_ERR_ARG;
  cudaError_t e = cudaFuncSetAttribute(project_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PJ_SMEM);
  if (e != cudaSuccess) return T2T_ERR_CUDA;
  dim3 grid(cdiv(N, PJ_ROWS), H);
  project_kernel<<<grid, 128, PJ_SMEM, stream>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)U,
                                                 (__nv_bfloat16*)out, N, x_row_stride, x_head_stride, d_status);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}

extern "C" int t2t_umma_selftest(const void* A, const void* B, const void* V, float* S_out, float* O_out,
                                 int* d_status, cudaStream_t stream) {
  using namespace t2t;
  if (!A || !B || !V || !S_out || !O_out) return T2T_ERR_ARG;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM);
  if (e != cudaSuccess) return T2T_ERR_CUDA;
  umma_selftest_kernel<<<1, 128, ST_SMEM, stream>>>((const __nv_bfloat16*)A, (const __nv_bfloat16*)B,
                                                    (const __nv_bfloat16*)V, S_out, O_out, d_status);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}
