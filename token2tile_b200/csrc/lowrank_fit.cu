// Projection fit: matched rank-32 projections Uq, Uk of one attention call.
//
// Replaces `online_u` of the reference operator (token2tile/operator/deploy_step.py:122-149;
// batched variants integrations/sglang/backend/t2t_attn.py:181-239), which runs two [N,128]^T[N,128]
// products per head in fp64 cuBLAS and three cuSOLVER factorisations per head from a Python loop.
// Here the whole fit is three kernels, batched over heads, with no host round trip:
//
//   gram_kernel        G = X^T X on the tcgen05 tensor cores.  One CTA takes a slab of up to 8192 rows
//                      of one head: 128-row tiles arrive by TMA (rows past N read as zeros) and serve
//                      as BOTH operands of a 128 x 128 x 128 product (A = tile^T, B = tile, both
//                      MN-major views of the same shared-memory tile); fp32 accumulator in TMEM.
//                      HBM-bound: every input row is read once.
//   sym_roots_kernel   sums the slabs in a fixed order in fp64 (M = G / N, deterministic), then finds
//                      M = V diag(e) V^T by one-sided Jacobi in shared memory and writes
//                      M^(1/2) (and M^(-1/2) for the query side) with the eigenvalues clamped at 1e-8.
//   lowrank_kernel     C = Mq^(1/2) Mk^(1/2), its singular triplets by one-sided Jacobi, the 32 largest:
//                      Uq = Mq^(-1/2) U_r S_r^(1/2),  Uk = Mk^(-1/2) V_r S_r^(1/2) = Mq^(1/2) U_r S_r^(-1/2)
//                      (V = C^T U S^-1 and Mk^(-1/2) Mk^(1/2) = I).
//
// One-sided (Hestenes) Jacobi orthogonalises the columns of W by plane rotations, W <- W J: for a
// symmetric positive semi-definite M the columns of the limit are e_i v_i, for a general C they are
// s_i u_i.  64 disjoint column pairs rotate per round (round-robin schedule, 127 rounds per sweep),
// 16 threads per pair, all in fp64.  Eigenvectors of clamped eigenvalues are never normalised:
// because every clamped eigenvalue has the same value c, their joint contribution to f(M) is
// f(c) (I - sum of the other v v^T), whatever basis spans them.
#include <cuda.h>

#include "common.cuh"
#include "internal.h"
#include "t2t_b200.h"

namespace t2t {

// ---------------------------------------------------------------------------
// Gram matrices
// ---------------------------------------------------------------------------
constexpr int GR_ROWS = 128;                 // rows per tile
constexpr int GR_SLAB_TILES = 64;            // tiles per CTA: 8192 rows in one fp32 accumulation
constexpr int GR_TILE = GR_ROWS * kD * 2;    // 32 KB
constexpr int GR_STAGES = 3;
constexpr int GR_SMEM = GR_STAGES * GR_TILE + 128 + 1024;

__host__ __device__ inline int gram_slabs(int N) { return cdiv(cdiv(N, GR_ROWS), GR_SLAB_TILES); }

__global__ void __launch_bounds__(128) gram_kernel(const __grid_constant__ CUtensorMap mapX, float* __restrict__ partial,
                                                   int N, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + GR_STAGES * GR_TILE);      // [GR_STAGES] tile landed
  uint64_t* freeb = full + GR_STAGES;                                          // [GR_STAGES] products that read it finished
  uint64_t* done = freeb + GR_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + GR_STAGES * GR_TILE + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + GR_STAGES * GR_TILE + 72);

  const int tid = threadIdx.x, warp = tid >> 5;
  const int slab = blockIdx.x, h = blockIdx.y, slabs = gridDim.x;
  const int tile0 = slab * GR_SLAB_TILES;
  const int ntiles = min(GR_SLAB_TILES, cdiv(N, GR_ROWS) - tile0);

  if (warp == 0) {
    tmem_alloc(tmem_slot, 128);
    tmem_relinquish();
  }
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < 2 * GR_STAGES + 1; ++i) mbar_init(full + i, 1);
    mbar_init_fence();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (tid == 0) {
    // ---- copies: two 64-column halves of a tile per stage ----
    for (int t = 0; t < ntiles; ++t) {
      const int st = t % GR_STAGES;
      if (t >= GR_STAGES && !mbar_wait(freeb + st, ((t / GR_STAGES) - 1) & 1, abort_flag)) break;
      mbar_arrive_expect_tx(full + st, GR_TILE);
      const uint32_t dst = base + st * GR_TILE;
      tma_load_tile3(dst, &mapX, 0, (tile0 + t) * GR_ROWS, h, full + st);
      tma_load_tile3(dst + GR_ROWS * 128, &mapX, 64, (tile0 + t) * GR_ROWS, h, full + st);
    }
  } else if (tid == 32) {
    // ---- products: G += tile^T tile, eight steps of 16 rows ----
    constexpr uint32_t idesc = make_idesc_bf16(128, 128, true, true);
    constexpr uint32_t dhi = sdesc_hi(1024);
    for (int t = 0; t < ntiles; ++t) {
      const int st = t % GR_STAGES;
      if (!mbar_wait(full + st, (t / GR_STAGES) & 1, abort_flag)) break;
      tc_fence_after();
      const uint32_t lo = sdesc_lo(base + st * GR_TILE, GR_ROWS * 128);
#pragma unroll
      for (int s = 0; s < 8; ++s)
        umma_ss_lo(tmem, lo + s * (2048 >> 4), lo + s * (2048 >> 4), dhi, idesc, (t > 0 || s > 0) ? 1u : 0u);
      umma_commit(freeb + st);
    }
    umma_commit(done);
  }
  __syncwarp();
  const bool ok = mbar_wait(done, 0, abort_flag);
  tc_fence_after();
  if (ok) {
    float* dst = partial + ((size_t)h * slabs + slab) * (kD * kD) + (size_t)tid * kD;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t v[32];
      tmem_ld32(tmem_addr(tmem, warp * 32, c * 32), v);
      tmem_wait_ld();
#pragma unroll
      for (int j = 0; j < 8; ++j)
        reinterpret_cast<uint4*>(dst + c * 32)[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    }
  } else if (tid == 0 && status) {
    atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 128);
}

// ---------------------------------------------------------------------------
// one-sided Jacobi on a 128 x 128 fp64 matrix in shared memory
// ---------------------------------------------------------------------------
constexpr int JD = 128;                  // matrix order
constexpr int JLD = JD + 1;              // column stride in doubles: an odd stride spreads the pairs over the banks
constexpr int J_THREADS = 1024;          // 64 pairs x 16 threads
constexpr int J_MAX_SWEEPS = 18;
constexpr int J_SMEM = JD * JLD * 8 + 2 * JD * 8 + 64;

__device__ __forceinline__ double shfl_xor_d(double v, int m) {
  return __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(v), m, 16),
                          __shfl_xor_sync(0xffffffffu, __double2loint(v), m, 16));
}

// Squared norms of the columns of W into nrm2[0..127] (every thread calls it).
__device__ void column_norms2(const double* W, double* nrm2) {
  const int tid = threadIdx.x, col = tid >> 3, sub = tid & 7;
  double acc = 0.0;
#pragma unroll
  for (int m = 0; m < 16; ++m) {
    const double x = W[col * JLD + sub + 8 * m];
    acc = fma(x, x, acc);
  }
  acc += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(acc), 4, 8), __shfl_xor_sync(0xffffffffu, __double2loint(acc), 4, 8));
  acc += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(acc), 2, 8), __shfl_xor_sync(0xffffffffu, __double2loint(acc), 2, 8));
  acc += __hiloint2double(__shfl_xor_sync(0xffffffffu, __double2hiint(acc), 1, 8), __shfl_xor_sync(0xffffffffu, __double2loint(acc), 1, 8));
  if (sub == 0) nrm2[col] = acc;
  __syncthreads();
}

// Rotates column pairs of W (column j at W + j * JLD) until all columns are mutually orthogonal
// to working precision.  Every thread of the 1024-thread CTA calls it.
__device__ void jacobi_orthogonalise(double* W, double* nrm2, int* flag) {
  const int tid = threadIdx.x, pi = tid >> 4, sub = tid & 15;
  __syncthreads();      // W was just written by other threads
  // columns whose squared norm is below (1e-14 of the largest column)^2 are numerically zero: rotating
  // them against each other never settles and changes nothing that is used
  column_norms2(W, nrm2);
  double big = 0.0;
  for (int j = 0; j < JD; ++j) big = fmax(big, nrm2[j]);
  const double tiny2 = 1.0e-28 * big;
  for (int sweep = 0; sweep < J_MAX_SWEEPS; ++sweep) {
    __syncthreads();
    if (tid == 0) *flag = 0;
    __syncthreads();
    bool rotated = false;
    for (int round = 0; round < JD - 1; ++round) {
      // round-robin pairing of 128 players: player 127 stays, the others move round a ring of 127
      int p, q;
      if (pi == 0) { p = JD - 1; q = round; }
      else { p = (round + pi) % (JD - 1); q = (round + (JD - 1) - pi) % (JD - 1); }
      double* wp = W + p * JLD;
      double* wq = W + q * JLD;
      double alpha = 0.0, beta = 0.0, gamma = 0.0;
#pragma unroll
      for (int m = 0; m < 8; ++m) {
        const double a = wp[sub + 16 * m], b = wq[sub + 16 * m];
        alpha = fma(a, a, alpha);
        beta = fma(b, b, beta);
        gamma = fma(a, b, gamma);
      }
#pragma unroll
      for (int d = 8; d > 0; d >>= 1) {
        alpha += shfl_xor_d(alpha, d);
        beta += shfl_xor_d(beta, d);
        gamma += shfl_xor_d(gamma, d);
      }
      // all 16 threads of the pair hold the same sums (xor reductions add in the same tree order)
      if (alpha > tiny2 && beta > tiny2 && gamma * gamma > 1.0e-27 * alpha * beta) {
        const double zeta = (beta - alpha) / (2.0 * gamma);
        const double t = (zeta >= 0.0 ? 1.0 : -1.0) / (fabs(zeta) + sqrt(1.0 + zeta * zeta));
        const double c = 1.0 / sqrt(1.0 + t * t), s = c * t;
#pragma unroll
        for (int m = 0; m < 8; ++m) {
          const double a = wp[sub + 16 * m], b = wq[sub + 16 * m];
          wp[sub + 16 * m] = c * a - s * b;
          wq[sub + 16 * m] = s * a + c * b;
        }
        rotated = true;
      }
      __syncthreads();
    }
    if (rotated) *flag = 1;
    __syncthreads();
    if (*flag == 0) break;
  }
  __syncthreads();
}

constexpr double kEigFloor = 1.0e-8;     // clamp of the reference (deploy_step.py:137-138)

// One CTA per second-moment matrix (blockIdx.x < H: query side, else key side).
//   roots    [2 H][128][128] fp64: M^(1/2)
//   invroots [H][128][128] fp64:   M^(-1/2), query side only
//   bad      [2 H] int: 1 when the matrix holds a non-finite value (non-finite input)
__global__ void __launch_bounds__(J_THREADS, 1) sym_roots_kernel(const float* __restrict__ partial, int slabs, int H,
                                                                 double inv_n, double* __restrict__ roots,
                                                                 double* __restrict__ invroots, int* __restrict__ bad) {
  extern __shared__ __align__(16) uint8_t jsm[];
  double* W = reinterpret_cast<double*>(jsm);
  double* nrm2 = W + JD * JLD;
  double* coef = nrm2 + JD;
  int* flag = reinterpret_cast<int*>(coef + JD);
  const int tid = threadIdx.x, m = blockIdx.x;

  // M = (sum of the slabs, in slab order) / N; symmetric, so rows can be read as columns
  const float* src = partial + (size_t)m * slabs * (JD * JD);
  bool finite = true;
  for (int e = tid; e < JD * JD; e += J_THREADS) {
    double acc = 0.0;
    for (int s = 0; s < slabs; ++s) acc += (double)src[(size_t)s * (JD * JD) + e];
    acc *= inv_n;
    finite = finite && isfinite(acc);
    W[(e >> 7) * JLD + (e & 127)] = acc;
  }
  const int any_bad = __syncthreads_or(finite ? 0 : 1);
  if (any_bad) {          // the host raises; nothing below would converge on NaNs
    if (tid == 0) bad[m] = 1;
    return;
  }
  if (tid == 0) bad[m] = 0;

  jacobi_orthogonalise(W, nrm2, flag);
  column_norms2(W, nrm2);
  // column i of W is e_i v_i: with l_i = max(e_i, floor),
  //   M^(1/2)  = sqrt(floor) I + sum_i (sqrt(l_i) - sqrt(floor)) v_i v_i^T
  //   M^(-1/2) = floor^(-1/2) I + sum_i (l_i^(-1/2) - floor^(-1/2)) v_i v_i^T
  // and v_i v_i^T = w_i w_i^T / e_i^2; the terms of clamped eigenvalues vanish.
  const bool want_inv = m < H;
  for (int pass = 0; pass < (want_inv ? 2 : 1); ++pass) {
    if (tid < JD) {
      const double e2 = nrm2[tid], e = sqrt(e2);
      double f = 0.0;
      if (e > kEigFloor) f = (pass == 0 ? sqrt(e) - sqrt(kEigFloor) : 1.0 / sqrt(e) - 1.0 / sqrt(kEigFloor)) / e2;
      coef[tid] = f;
    }
    __syncthreads();
    const int col = tid & 127, r0 = (tid >> 7) * 16;      // 16 rows x 1 column per thread
    double acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0;
    for (int k = 0; k < JD; ++k) {
      const double f = coef[k] * W[k * JLD + col];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = fma(f, W[k * JLD + r0 + i], acc[i]);
    }
    const double diag = pass == 0 ? sqrt(kEigFloor) : 1.0 / sqrt(kEigFloor);
    double* dst = pass == 0 ? roots + (size_t)m * JD * JD : invroots + (size_t)m * JD * JD;
#pragma unroll
    for (int i = 0; i < 16; ++i) dst[(size_t)(r0 + i) * JD + col] = acc[i] + (r0 + i == col ? diag : 0.0);
    __syncthreads();
  }
}

// One CTA per head.  Uq, Uk fp32 [H][128][32].
__global__ void __launch_bounds__(J_THREADS, 1) lowrank_kernel(const double* __restrict__ roots,
                                                               const double* __restrict__ invroots, int H,
                                                               const int* __restrict__ bad, float* __restrict__ Uq,
                                                               float* __restrict__ Uk) {
  extern __shared__ __align__(16) uint8_t jsm[];
  double* W = reinterpret_cast<double*>(jsm);
  double* nrm2 = W + JD * JLD;
  double* coef = nrm2 + JD;                 // reused: the column chosen for each of the 32 ranks
  int* flag = reinterpret_cast<int*>(coef + JD);
  const int tid = threadIdx.x, h = blockIdx.x;
  if (bad[h] | bad[H + h]) return;
  const double* Rq = roots + (size_t)h * JD * JD;
  const double* Rk = roots + (size_t)(H + h) * JD * JD;
  const double* Rqi = invroots + (size_t)h * JD * JD;

  // C = Rq^T Rk = Rq Rk (both symmetric); column j of C goes to W + j * JLD
  {
    const int col = tid & 127, r0 = (tid >> 7) * 16;
    double acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.0;
    for (int k = 0; k < JD; ++k) {
      const double b = Rk[(size_t)k * JD + col];
#pragma unroll
      for (int i = 0; i < 16; ++i) acc[i] = fma(Rq[(size_t)(r0 + i) * JD + k], b, acc[i]);
    }
#pragma unroll
    for (int i = 0; i < 16; ++i) W[col * JLD + r0 + i] = acc[i];
  }
  jacobi_orthogonalise(W, nrm2, flag);
  column_norms2(W, nrm2);      // column j is s_j u_j

  // rank of every column by decreasing singular value (ties: lower column first)
  int* pick = reinterpret_cast<int*>(coef);
  if (tid < JD) {
    const double mine = nrm2[tid];
    int rank = 0;
    for (int j = 0; j < JD; ++j) {
      const double o = nrm2[j];
      rank += (o > mine || (o == mine && j < tid)) ? 1 : 0;
    }
    if (rank < kR) pick[rank] = tid;
  }
  __syncthreads();
  // Uq[:, r] = Rqi w / sqrt(s),  Uk[:, r] = Rq w / s^(3/2)     (w = s u, the chosen column)
  for (int e = tid; e < JD * kR; e += J_THREADS) {
    const int d = e >> 5, r = e & 31, j = pick[r];
    const double s2 = nrm2[j], s = sqrt(s2);
    double aq = 0.0, ak = 0.0;
    for (int k = 0; k < JD; ++k) {
      const double w = W[j * JLD + k];
      aq = fma(Rqi[(size_t)d * JD + k], w, aq);
      ak = fma(Rq[(size_t)d * JD + k], w, ak);
    }
    const bool live = s > 0.0;
    Uq[((size_t)h * JD + d) * kR + r] = live ? (float)(aq / sqrt(s)) : 0.f;
    Uk[((size_t)h * JD + d) * kR + r] = live ? (float)(ak / (s * sqrt(s))) : 0.f;
  }
}

}  // namespace t2t

using namespace t2t;

static size_t fit_off_roots(int H, int N) { return (((size_t)2 * H * gram_slabs(N) * kD * kD * 4) + 255) & ~(size_t)255; }
static size_t fit_off_inv(int H, int N) { return fit_off_roots(H, N) + (size_t)2 * H * kD * kD * 8; }

extern "C" size_t t2t_lowrank_fit_ws_bytes(int H, int N) { return fit_off_inv(H, N) + (size_t)H * kD * kD * 8; }

extern "C" int t2t_lowrank_fit(const void* q, const void* k, float* Uq, float* Uk, int H, int N, void* ws,
                               size_t ws_bytes, int* d_bad, int* d_status, cudaStream_t st) {
  return t2t_lowrank_fit_strided(q, k, (long long)kD, (long long)N * kD, Uq, Uk, H, N, ws, ws_bytes, d_bad, d_status,
                                 st);
}

extern "C" int t2t_lowrank_fit_strided(const void* q, const void* k, long long row_stride, long long head_stride,
                                       float* Uq, float* Uk, int H, int N, void* ws, size_t ws_bytes, int* d_bad,
                                       int* d_status, cudaStream_t st) {
  if (!q || !k || !Uq || !Uk || !ws || !d_bad || H <= 0 || N <= 0) return T2T_ERR_ARG;
  if (row_stride < kD || head_stride <= 0) return T2T_ERR_ARG;
  if (ws_bytes < t2t_lowrank_fit_ws_bytes(H, N)) return T2T_ERR_WORKSPACE;
  char* w = static_cast<char*>(ws);
  float* partial = reinterpret_cast<float*>(w);
  double* roots = reinterpret_cast<double*>(w + fit_off_roots(H, N));
  double* invroots = reinterpret_cast<double*>(w + fit_off_inv(H, N));
  const int slabs = gram_slabs(N);
  if (cudaFuncSetAttribute(gram_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, GR_SMEM) != cudaSuccess ||
      cudaFuncSetAttribute(sym_roots_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, J_SMEM) != cudaSuccess ||
      cudaFuncSetAttribute(lowrank_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, J_SMEM) != cudaSuccess)
    return T2T_ERR_CUDA;
  CUtensorMap mq, mk;
  if (!make_head_tile_map(&mq, q, (uint64_t)N, (uint64_t)H, GR_ROWS, (uint64_t)row_stride, (uint64_t)head_stride) ||
      !make_head_tile_map(&mk, k, (uint64_t)N, (uint64_t)H, GR_ROWS, (uint64_t)row_stride, (uint64_t)head_stride))
    return T2T_ERR_CUDA;
  gram_kernel<<<dim3(slabs, H), 128, GR_SMEM, st>>>(mq, partial, N, d_status);
  gram_kernel<<<dim3(slabs, H), 128, GR_SMEM, st>>>(mk, partial + (size_t)H * slabs * kD * kD, N, d_status);
  sym_roots_kernel<<<2 * H, J_THREADS, J_SMEM, st>>>(partial, slabs, H, 1.0 / (double)N, roots, invroots, d_bad);
  lowrank_kernel<<<H, J_THREADS, J_SMEM, st>>>(roots, invroots, H, d_bad, Uq, Uk);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}
