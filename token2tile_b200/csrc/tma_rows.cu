// Tensor maps for row gathers and their self-test.
//
// The attention kernel reads K and V tiles whose 128 rows are scattered runs of a
// cluster-major matrix.  A tensor map with a (64 columns x 1 row) box lets one TMA
// instruction fetch four arbitrary rows into four consecutive rows of a
// SWIZZLE_128B tile, which is the operand layout tcgen05.mma reads.
#include <cuda.h>

#include "common.cuh"
#include "internal.h"

namespace t2t {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up once per process (it does not depend on the device).
static EncodeTiledFn encode_tiled() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

bool make_row_tile_map(void* map_out, const void* base, uint64_t rows, uint32_t box_rows) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn || (reinterpret_cast<uintptr_t>(base) & 15u) || box_rows == 0 || box_rows > 256) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)kD, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kD * 2};
  const cuuint32_t box[2] = {64, box_rows};
  const cuuint32_t elem[2] = {1, 1};
  return fn(reinterpret_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
            dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_head_tile_map(void* map_out, const void* base, uint64_t rows_per_head, uint64_t heads, uint32_t box_rows,
                        uint64_t row_stride, uint64_t head_stride) {
  EncodeTiledFn fn = encode_tiled();
  if (!fn || (reinterpret_cast<uintptr_t>(base) & 15u) || box_rows == 0 || box_rows > 256) return false;
  if ((row_stride & 7u) || (head_stride & 7u)) return false;      // TMA strides are multiples of 16 bytes
  const cuuint64_t dims[3] = {(cuuint64_t)kD, (cuuint64_t)rows_per_head, (cuuint64_t)heads};
  const cuuint64_t strides[2] = {(cuuint64_t)row_stride * 2, (cuuint64_t)head_stride * 2};
  const cuuint32_t box[3] = {64, box_rows, 1};
  const cuuint32_t elem[3] = {1, 1, 1};
  return fn(reinterpret_cast<CUtensorMap*>(map_out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
            dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_row_gather_map(void* map_out, const void* base, uint64_t rows) {
  return make_row_tile_map(map_out, base, rows, 1);
}

// One 128-row tile gathered by 64 instructions (two 64-column blocks x 32 groups of
// four rows), copied back to global memory byte for byte.
__global__ void __launch_bounds__(128) gather4_selftest_kernel(const __grid_constant__ CUtensorMap map,
                                                               const int* __restrict__ gidx,
                                                               uint4* __restrict__ out, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bar = reinterpret_cast<uint64_t*>(sm + 32768);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + 32768 + 16);
  const int tid = threadIdx.x;
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(bar, 1);
    mbar_init_fence();
  }
  __syncthreads();
  if (tid == 0) mbar_arrive_expect_tx(bar, 32768);
  if (tid < 64) {
    const int b = tid >> 5, g = tid & 31;
    const int4 r = reinterpret_cast<const int4*>(gidx)[g];
    tma_gather4(base + b * 16384 + g * 512, &map, b * 64, r.x, r.y, r.z, r.w, bar);
  }
  const bool ok = mbar_wait(bar, 0, abort_flag);
  if (ok) {
    for (int i = tid; i < 2048; i += 128) out[i] = reinterpret_cast<const uint4*>(sm)[i];
  } else if (tid == 0 && status) {
    atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
  }
}

// The give-up path of the bounded waits, exercised on purpose: a barrier that nobody arrives on, a
// short spin limit, and the same exit sequence as the production kernels (raise the abort flag, report
// through the status word, return).  The kernel always terminates.
__global__ void __launch_bounds__(64) wait_timeout_selftest_kernel(int* __restrict__ status, int* __restrict__ out) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int tid = threadIdx.x;
  if (tid == 0) {
    abort_word = 0;
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  __syncthreads();
  // warp 0 runs into the limit; warp 1 starts later and leaves as soon as it sees the abort flag
  bool ok;
  if (tid < 32) {
    ok = mbar_wait_limited(&bar, 0, abort_flag, 1u << 10);
  } else {
    ok = mbar_wait_limited(&bar, 0, abort_flag, kWaitSpinLimit);
  }
  if (tid == 0 || tid == 32) out[tid >> 5] = ok ? 1 : 0;
  __syncthreads();
  if (tid == 0 && *abort_flag) atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
}

}  // namespace t2t

using namespace t2t;

extern "C" int t2t_wait_timeout_selftest(int* d_status, int* d_out, cudaStream_t st) {
  if (!d_status || !d_out) return T2T_ERR_ARG;
  wait_timeout_selftest_kernel<<<1, 64, 0, st>>>(d_status, d_out);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}

extern "C" int t2t_gather4_selftest(const void* src, int rows, const int* gidx, void* out, int* d_status,
                                    cudaStream_t st) {
  if (!src || !gidx || !out || rows <= 0) return T2T_ERR_ARG;
  CUtensorMap map;
  if (!make_row_gather_map(&map, src, (uint64_t)rows)) return T2T_ERR_CUDA;
  const int smem = 32768 + 64 + 1024;
  gather4_selftest_kernel<<<1, 128, smem, st>>>(map, gidx, reinterpret_cast<uint4*>(out), d_status);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}
