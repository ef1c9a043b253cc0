// Task plan, packed exact tile attention and centroid residual + merge.
//
// Replaces the reference's tile_attn extension
// (token2tile/operator/kernels/tile_attn/src/kernel.cu: selected_kv_lengths,
// plan_kernel, attn_kernel, tail_wgmma_kernel), whose wgmma kernels do not
// exist on sm_100a.  Both hot kernels run their matrix products on the
// tcgen05 tensor cores with fp32 accumulators in tensor memory (TMEM):
//
//   attention:  S = Q K^T   (128 queries x 128 keys, K = 128)   operands in smem
//               O += P V    (P = exp2(S - m) as bf16 in TMEM, V in smem)
//   residual :  S = QU cks^T (128 queries x 128 centroids, K = 32)
//               T += P sumv (128 x 128, K = 128 centroids)
//
// One thread owns one query row (TMEM lane), so row maxima and sums need no
// shuffles.  K/V rows of a union are contiguous runs in the cluster-major
// copies kp/vp; the attention kernels fetch them with TMA row gathers (four
// rows per instruction) straight into 128-byte-swizzled tiles, the residual
// kernel with 16-byte cp.async.  Tasks of up to 128 query rows run in
// attn_kernel, two CTAs to an SM (256 TMEM columns each) so that the softmax
// of one overlaps the MMAs and loads of the other; tasks of 129..256 rows run
// in attn2_kernel, one warp-specialised CTA per SM whose two row groups share
// one K/V stream.  Every mbarrier wait is bounded; on a timeout the CTA raises
// a status word and leaves.
#include <cuda.h>

#include <mutex>

#include "common.cuh"
#include "internal.h"
#include "t2t_b200.h"

namespace t2t {

constexpr int QT = 128;          // query rows per tensor-core tile (one thread per row)
constexpr int TASK_ROWS = 256;   // query rows per task: tasks above QT rows run as two tiles sharing one K/V stream
constexpr int KT = 128;          // keys per tile
constexpr int MAX_RUNS = 1024;   // runs of selected clusters in one union
constexpr int PLAN_SORT_MAX = 2048;
constexpr int PLAN_HDR = 8;      // counters: [0] tasks, [1] cursor of the one-tile kernel, [2..3] executed pairs (lo, hi),
                                 //           [4] cursor of the two-tile kernel

// Layout of the plan (an int32 array owned by a structure snapshot): first row of every key cluster in kp / vp,
// one bit per key cluster saying whether it holds any token, the counters (on a 16-byte boundary: the pair
// count is a 64-bit atomic), the tasks, and the union length of every query cluster.
__host__ __device__ inline size_t plan_nonempty_offset(int H) { return (size_t)H * (kC + 1); }
__host__ __device__ inline size_t plan_counter_offset(int H) { return (plan_nonempty_offset(H) + (size_t)H * (kC / 32) + 3) & ~(size_t)3; }
__host__ __device__ inline size_t plan_task_offset(int H) { return plan_counter_offset(H) + PLAN_HDR; }
__host__ __device__ inline size_t plan_max_tasks(int H, int N, int CQ) { return (size_t)H * (CQ + cdiv(N, TASK_ROWS) + 1); }

struct PlanView {
  int* k_off;           // [H][C + 1]
  uint32_t* nonempty;   // [H][C / 32]
  int* counters;        // [PLAN_HDR]
  int4* tasks;          // (head, query cluster, first sorted row, rows)
  int* kv_lens;         // [H][CQ]
};
__host__ __device__ inline PlanView plan_view(int* plan, int H, int N, int CQ) {
  PlanView v;
  v.k_off = plan;
  v.nonempty = reinterpret_cast<uint32_t*>(plan + plan_nonempty_offset(H));
  v.counters = plan + plan_counter_offset(H);
  v.tasks = reinterpret_cast<int4*>(plan + plan_task_offset(H));
  v.kv_lens = plan + plan_task_offset(H) + 4 * plan_max_tasks(H, N, CQ);
  return v;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---------------------------------------------------------------------------
// plan: key-cluster offsets, union lengths, tasks (most work first inside a head)
// ---------------------------------------------------------------------------
// Exclusive prefix of v over the 256 threads of the CTA (every thread calls it); scratch holds 8 ints.
__device__ __forceinline__ int block_prefix_256(int v, int* scratch, int& total) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int inc = warp_incl_scan(v, lane);
  __syncthreads();
  if (lane == 31) scratch[w] = inc;
  __syncthreads();
  int before = 0, all = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int part = scratch[i];
    before += i < w ? part : 0;
    all += part;
  }
  total = all;
  return before + inc - v;
}

// One CTA per head.  A query cluster of n rows gives ceil(n / TASK_ROWS) tasks: full ones first, the remainder
// last (a remainder of at most QT rows costs one row tile instead of two).
__global__ void __launch_bounds__(256) plan_kernel(const int* __restrict__ qcount, const int* __restrict__ kcount,
                                                   const uint32_t* __restrict__ ubits, int H, int N, int CQ,
                                                   int* __restrict__ plan) {
  __shared__ int s_off[kC + 1];
  __shared__ unsigned long long s_key[PLAN_SORT_MAX];
  __shared__ int s_scan[8];
  const PlanView pv = plan_view(plan, H, N, CQ);
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  // first kp / vp row of every key cluster (eight consecutive clusters per thread) and the non-empty bits
  {
    int c8[8], sum = 0;
    uint32_t some = 0u;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      c8[i] = kcount[(size_t)h * kC + tid * 8 + i];
      sum += c8[i];
      some |= (c8[i] > 0 ? 1u : 0u) << i;
    }
    int total;
    int run = block_prefix_256(sum, s_scan, total);
#pragma unroll
    for (int i = 0; i < 8; ++i) { s_off[tid * 8 + i] = run; run += c8[i]; }
    if (tid == 255) s_off[kC] = run;
    // four neighbouring threads hold the four bytes of one 32-cluster word
    uint32_t word = some << (8 * (tid & 3));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if ((tid & 3) == 0) pv.nonempty[(size_t)h * (kC / 32) + (tid >> 2)] = word;
  }
  __syncthreads();
  for (int i = tid; i <= kC; i += 256) pv.k_off[(size_t)h * (kC + 1) + i] = s_off[i];

  // tokens in the union of every query cluster (a warp per cluster), and the pairs the head executes
  unsigned long long pairs = 0;
  for (int c = warp; c < CQ; c += 8) {
    const int n = qcount[(size_t)h * CQ + c];
    int len = 0;
    if (n > 0) {
      const uint32_t* words = ubits + ((size_t)h * CQ + c) * (kC / 32);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int w = lane + 32 * half;
        for (uint32_t bits = words[w]; bits; bits &= bits - 1) {
          const int cl = w * 32 + __ffs(bits) - 1;
          len += s_off[cl + 1] - s_off[cl];
        }
      }
    }
    len = __reduce_add_sync(0xffffffffu, len);
    if (lane == 0) {
      pv.kv_lens[(size_t)h * CQ + c] = len;
      pairs += (unsigned long long)n * (unsigned long long)len;
    }
  }
  if (lane == 0 && pairs) atomicAdd(reinterpret_cast<unsigned long long*>(pv.counters + 2), pairs);
  __syncthreads();

  // the task array is head-major (the K / V rows of a head stay in L2 while its unions are read):
  // count the tasks of the heads before this one
  int first = 0, mine = 0;
  for (int hh = 0; hh <= h; ++hh) {
    int cnt = 0;
    for (int c = tid; c < CQ; c += 256) cnt += cdiv(qcount[(size_t)hh * CQ + c], TASK_ROWS);
    int total;
    block_prefix_256(cnt, s_scan, total);
    if (hh < h) first += total; else mine = total;
  }
  if (h == H - 1 && tid == 0) pv.counters[0] = first + mine;

  int rows_before = 0, tasks_before = 0;
  for (int c0 = 0; c0 < CQ; c0 += 256) {
    const int c = c0 + tid;
    const int n = c < CQ ? qcount[(size_t)h * CQ + c] : 0;
    const int nt = cdiv(n, TASK_ROWS);
    int tot_rows, tot_tasks;
    const int row0 = rows_before + block_prefix_256(n, s_scan, tot_rows);
    const int task0 = tasks_before + block_prefix_256(nt, s_scan, tot_tasks);
    for (int i = 0; i < nt; ++i)
      pv.tasks[first + task0 + i] = make_int4(h, c, row0 + i * TASK_ROWS, min(TASK_ROWS, n - i * TASK_ROWS));
    rows_before += tot_rows;
    tasks_before += tot_tasks;
  }
  __syncthreads();
  if (mine < 2 || mine > PLAN_SORT_MAX) return;

  // most work first (rows x union length); equal work keeps its order
  int pow2 = 2;
  while (pow2 < mine) pow2 <<= 1;
  for (int i = tid; i < pow2; i += 256) {
    unsigned long long key = 0ull;
    if (i < mine) {
      const int4 t = pv.tasks[first + i];
      const unsigned long long work = min((unsigned long long)t.w * (unsigned long long)pv.kv_lens[(size_t)h * CQ + t.y], 0xFFFFFFFFull);
      key = (work << 32) | (unsigned long long)(0xFFFFFFFFu - (unsigned)i);
    }
    s_key[i] = key;
  }
  __syncthreads();
  for (int span = 2; span <= pow2; span <<= 1) {
    for (int step = span >> 1; step > 0; step >>= 1) {
      for (int i = tid; i < pow2; i += 256) {
        const int j = i ^ step;
        if (j > i) {
          const unsigned long long x = s_key[i], y = s_key[j];
          const bool descending = (i & span) == 0;
          if (descending ? x < y : x > y) { s_key[i] = y; s_key[j] = x; }
        }
      }
      __syncthreads();
    }
  }
  int4 keep[PLAN_SORT_MAX / 256];
  int k = 0;
  for (int i = tid; i < mine; i += 256) keep[k++] = pv.tasks[first + (int)(0xFFFFFFFFu - (unsigned)(s_key[i] & 0xFFFFFFFFull))];
  __syncthreads();
  k = 0;
  for (int i = tid; i < mine; i += 256) pv.tasks[first + i] = keep[k++];
}

__global__ void plan_info_kernel(const int* __restrict__ counters, int* __restrict__ info) {
  if (threadIdx.x < 4) info[threadIdx.x] = threadIdx.x == 0 ? counters[0] : (threadIdx.x < 3 ? counters[threadIdx.x + 1] : 0);
}

// ---------------------------------------------------------------------------
// shared pieces of the two tensor-core kernels
// ---------------------------------------------------------------------------
struct RowState {
  float m;      // reference maximum (log2 domain) the stored P and O are relative to
  float l;      // running denominator
};

constexpr float kLazy = 8.0f;   // rescale O only when the row maximum grows by more than 2^8

// Rescale the fp32 accumulator rows in TMEM by `alpha` (per thread = per row).
__device__ __forceinline__ void rescale_rows(uint32_t tO_lane, float alpha) {
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld32(tO_lane + c * 32, v);
    tmem_wait_ld();
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * alpha);
    tmem_st32(tO_lane + c * 32, v);
  }
}

// The union of one task as runs of consecutive kp / vp rows: maximal stretches of selected, non-empty key
// clusters that follow each other.  sRunStart[r] = first row of run r, sRunCum[r] = position of its first
// token in the union, sRunCum[runs] = union length, *runs_out = runs.  One warp does the work with the bitmap
// as 64-bit words (two bitmap words per lane): a run starts at a set bit whose lower neighbour is clear and
// ends at a set bit whose upper neighbour is clear, so the r-th start and the r-th end delimit run r.  A run
// list that would not fit raises the abort flag.
__device__ __forceinline__ void build_runs_warp(const int* __restrict__ koh, const uint32_t* __restrict__ ubr,
                                                const uint32_t* __restrict__ nonempty, int* sRunStart, int* sRunCum,
                                                int* runs_out, volatile int* abort_flag, int* status) {
  const int lane = threadIdx.x & 31;
  const unsigned long long sel = ((unsigned long long)(ubr[2 * lane + 1] & nonempty[2 * lane + 1]) << 32) |
                                 (unsigned long long)(ubr[2 * lane] & nonempty[2 * lane]);
  // neighbours across the lane boundary
  const unsigned long long below = __shfl_up_sync(0xffffffffu, sel, 1), above = __shfl_down_sync(0xffffffffu, sel, 1);
  const unsigned long long carry_in = lane > 0 ? below >> 63 : 0ull;
  const unsigned long long carry_out = lane < 31 ? (above & 1ull) << 63 : 0ull;
  unsigned long long starts = sel & ~((sel << 1) | carry_in);
  unsigned long long ends = sel & ~((sel >> 1) | carry_out);
  const int mine = __popcll(starts);
  const int before_s = warp_incl_scan(mine, lane) - mine;
  const int before_e = warp_incl_scan(__popcll(ends), lane) - __popcll(ends);
  const int runs = __shfl_sync(0xffffffffu, before_s + mine, 31);
  if (runs > MAX_RUNS) {      // cannot happen for C = 2048; guard the static arrays anyway
    if (lane == 0) { *abort_flag = 1; if (status) atomicExch(status, ST_BAD_PLAN); }
    return;
  }
  int r = before_s;
  for (; starts; starts &= starts - 1) sRunStart[r++] = koh[64 * lane + __ffsll((long long)starts) - 1];
  r = before_e;
  for (; ends; ends &= ends - 1) sRunCum[r++] = koh[64 * lane + __ffsll((long long)ends)];      // one past the run's last row
  __syncwarp();
  // lengths -> positions: every lane turns a block of consecutive runs into a running sum
  const int per = (runs + 31) >> 5, lo = min(lane * per, runs), hi = min(lo + per, runs);
  int sum = 0;
  for (int i = lo; i < hi; ++i) sum += sRunCum[i] - sRunStart[i];
  int pos = warp_incl_scan(sum, lane) - sum;
  const int total = __shfl_sync(0xffffffffu, pos + sum, 31);
  for (int i = lo; i < hi; ++i) {
    const int len = sRunCum[i] - sRunStart[i];
    sRunCum[i] = pos;
    pos += len;
  }
  if (lane == 0) { sRunCum[runs] = total; *runs_out = runs; }
}
// The same for a whole CTA: warp 0 builds the list into sMisc[1], a CTA-wide barrier publishes it.  Returns
// false when the list would not fit (the abort flag is then set).
__device__ __forceinline__ bool build_runs(const int* __restrict__ koh, const uint32_t* __restrict__ ubr,
                                           const uint32_t* __restrict__ nonempty, int* sRunStart, int* sRunCum,
                                           int* sMisc, volatile int* abort_flag, int* status) {
  if ((threadIdx.x >> 5) == 0) build_runs_warp(koh, ubr, nonempty, sRunStart, sRunCum, sMisc + 1, abort_flag, status);
  __syncthreads();
  return *abort_flag == 0;
}

constexpr int AT_TILE = KT * kD * 2;   // 32 KB: one 128-row tile of q, kp or vp

// kp / vp rows (all heads: `row0` is the head's first row) of union positions p0 .. p0 + 3, from the run list of
// build_runs.  `cursor` is the caller's run index from its previous, smaller p0 (0 at the start of a task): the
// run of p0 is found by stepping forward from it.  Positions past the union read the head's first row (their
// scores are masked).  Returns whether the four rows exist and are consecutive rows of kp / vp.
__device__ __forceinline__ bool union_rows(const int* sRunStart, const int* sRunCum, int nruns, int kvlen, int p0,
                                           int row0, int& cursor, int (&r)[4]) {
  int ru = cursor;
  while (ru + 1 < nruns && sRunCum[ru + 1] <= p0) ++ru;
  cursor = ru;
  int next = sRunCum[ru + 1];
  int row = sRunStart[ru] + p0 - sRunCum[ru];
  r[0] = p0 < kvlen ? row0 + row : row0;
#pragma unroll
  for (int j = 1; j < 4; ++j) {
    const int p = p0 + j;
    if (p >= next && ru + 1 < nruns) {
      ++ru;
      row = sRunStart[ru];
      next = sRunCum[ru + 1];
    } else {
      ++row;
    }
    r[j] = p < kvlen ? row0 + row : row0;
  }
  return p0 + 3 < kvlen && r[3] == r[0] + 3;
}

// Tensor maps over kp and vp as [H * N, 128] matrices with boxes of 1, 32 and 64 rows by 64 columns.
struct KVMaps {
  CUtensorMap k1, k32, k64, v1, v32, v64;
};

// How a warp fetches a 128-row K or V tile.  Lane g owns destination rows 4 g .. 4 g + 3, whose source rows are
// r[0..3]; `whole` says that they are four consecutive rows of kp / vp.  Groups that follow each other in the
// source as well form a stretch, and a stretch is fetched with 64-row tile loads, then 32-row tile loads, then
// four-row gathers for what is left (a tile load moves 2.6x / 1.8x the bytes per cycle of a gather; a swizzled
// tile may start at any multiple of four rows, the pattern being a function of the shared-memory address).
// Groups that straddle two runs of the union are gathered.  Returns what this lane issues for each 64-column
// block: FETCH_NONE (a tile load of a lower lane covers its rows), a gather, or a tile load starting at r[0].
enum { FETCH_NONE = 0, FETCH_GATHER = 1, FETCH_BOX32 = 2, FETCH_BOX64 = 3 };
__device__ __forceinline__ int fetch_plan(const int (&r)[4], bool whole, int lane) {
  const int prev = __shfl_up_sync(0xffffffffu, r[0], 1);
  const unsigned wmask = __ballot_sync(0xffffffffu, whole);
  const bool linked = whole && lane > 0 && ((wmask >> (lane - 1)) & 1u) && r[0] == prev + 4;
  const unsigned lmask = __ballot_sync(0xffffffffu, linked);      // bit g: group g continues the stretch of g - 1
  if (!whole) return FETCH_GATHER;
  const unsigned upto = 0xffffffffu >> (31 - lane);
  const int start = 31 - __clz((wmask & ~lmask) & upto);
  const unsigned above = ~lmask & ~upto;
  const int end = above ? __ffs(above) - 1 : 32;
  const int len = end - start, k = lane - start;
  const int k64 = len & ~15, k32 = k64 + ((len - k64) & ~7);
  if (k < k64) return (k & 15) == 0 ? FETCH_BOX64 : FETCH_NONE;
  if (k < k32) return ((k - k64) & 7) == 0 ? FETCH_BOX32 : FETCH_NONE;
  return FETCH_GATHER;
}
// One lane's part of one 64-column block (`dst`: the block's first byte; bytes are counted on `full`).
__device__ __forceinline__ void fetch_issue(int what, uint32_t dst, const CUtensorMap* map1, const CUtensorMap* map32,
                                            const CUtensorMap* map64, int col, const int (&r)[4], int lane,
                                            uint64_t* full) {
  const uint32_t mine = dst + lane * 512;
  if (what == FETCH_GATHER) tma_gather4(mine, map1, col, r[0], r[1], r[2], r[3], full);
  else if (what == FETCH_BOX32) tma_load_tile(mine, map32, col, r[0], full);
  else if (what == FETCH_BOX64) tma_load_tile(mine, map64, col, r[0], full);
}

// ---------------------------------------------------------------------------
// exact attention, tasks of QT + 1 .. TASK_ROWS rows
// ---------------------------------------------------------------------------
// Two row tiles share one K/V stream, so the union crosses L2 -> SM once per task
// instead of once per 128 rows, and the roles are separated so that nobody who
// computes ever waits on an issue queue:
//   warps 0..3 / 4..7  softmax of row group 0 / 1: one thread per query row; S / P
//                      and O of a group live in its own half of tensor memory
//   warp 8             one lane issues every MMA (an MMA blocks its issuer while the
//                      tensor pipe's queue is full)
//   warps 10..15       stream K and V tiles into two-slot rings with four-row TMA gathers.
//                      A gather blocks its warp for about 70 cycles per lane, one lane at a
//                      time, but gathers of different warps overlap: six warps issue the
//                      128 gathers of a tile pair, 21 or 22 each
//   (warp 9 only takes part in the CTA-wide barriers: 16 warps keep four per scheduler)
// Hand-offs are mbarriers: S[g] / O[g] (MMA done -> softmax), P[g] (softmax -> MMA),
// fullK / fullV[s] (copy landed -> MMA), freeK / freeV[s] (both groups' MMA done -> copy: one
// commit after group 1's MMA, which the tensor pipe runs after group 0's),
// fullQ[g].  Ring slot s holds tile g with g & 1 == s, where g counts the tiles this
// CTA has processed; the n-th fill of a slot waits for phase n of its free barrier
// (phase 0 is completed at start-up) and completes phase n of its full barrier.
// Packed fp32 pairs (one instruction for two values) and the three-input maximum keep the instruction count of
// the softmax rows down: the MMA lane and the copy warps share their schedulers.
__device__ __forceinline__ unsigned long long pack_f2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f2(unsigned long long v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_f2(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ unsigned long long add_f2(unsigned long long a, unsigned long long b) {
  unsigned long long r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// 2^y for two values y <= 8 without the special-function unit: round y to the nearest integer n (the
// magic-number add leaves n in the low mantissa bits), a cubic for 2^(y - n) on [-0.5, 0.5] (relative error
// 7.5e-5, well inside a bf16 rounding step), and n added to the exponent field.  Inputs below -125 count as
// -125 (2^-125 ~ 0).
__device__ __forceinline__ void exp2_fma2(float y0, float y1, float& p0, float& p1) {
  const unsigned long long y = pack_f2(fmaxf(y0, -125.0f), fmaxf(y1, -125.0f));
  const unsigned long long t = add_f2(y, pack_f2(12582912.0f, 12582912.0f));      // 1.5 * 2^23
  const unsigned long long n = add_f2(t, pack_f2(-12582912.0f, -12582912.0f));
  const unsigned long long f = fma_f2(n, pack_f2(-1.0f, -1.0f), y);
  unsigned long long p = fma_f2(pack_f2(0.055171408f, 0.055171408f), f, pack_f2(0.24261075f, 0.24261075f));
  p = fma_f2(p, f, pack_f2(0.69326097f, 0.69326097f));
  p = fma_f2(p, f, pack_f2(0.99992812f, 0.99992812f));
  float q0, q1, t0, t1;
  unpack_f2(p, q0, q1);
  unpack_f2(t, t0, t1);
  p0 = __int_as_float(__float_as_int(q0) + (__float_as_int(t0) << 23));
  p1 = __int_as_float(__float_as_int(q1) + (__float_as_int(t1) << 23));
}

// Softmax of one 128-column S row held in tensor memory, in two passes of 32-column chunks so that few
// registers are live: the row maximum first, then P = 2^(s * scale - m) packed to bf16 over the columns S
// occupied (chunk c of S, columns 32 c .., becomes columns 16 c .. of P: always columns that were read
// before).  Two row groups that compute at the same time are bound by the special-function unit (16
// exponentials per cycle and SM), so every third pair of a full tile takes the FMA-pipe route instead.
// MASK: columns >= valid lie past the union and count as -inf (all of them through the special-function
// unit, whose result for -inf is an exact zero).
constexpr int kFmaPairEvery = 3;
// `halfway` is called by the whole warp once the first 64 columns of P are written, so that the MMA lane can
// start on them while the rows work on the rest.
template <bool MASK, typename Halfway>
__device__ __forceinline__ void softmax_tile(uint32_t tS_lane, uint32_t tO_lane, RowState& rs, int valid, bool first,
                                             float sc, Halfway&& halfway) {
  float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld32(tS_lane + c * 32, v);
    tmem_wait_ld();
    if (MASK) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c * 32 + j >= valid) v[j] = 0xff800000u;      // -inf
    }
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      mx4[0] = max3(mx4[0], __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
      mx4[1] = max3(mx4[1], __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      mx4[2] = max3(mx4[2], __uint_as_float(v[j + 4]), __uint_as_float(v[j + 5]));
      mx4[3] = max3(mx4[3], __uint_as_float(v[j + 6]), __uint_as_float(v[j + 7]));
    }
  }
  const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * sc;
  if (first) {
    rs.m = mx;
  } else {
    const bool grow = mx > rs.m + kLazy;
    if (__any_sync(0xffffffffu, grow)) {
      const float mnew = grow ? mx : rs.m;
      const float alpha = ex2_approx(rs.m - mnew);
      rescale_rows(tO_lane, alpha);
      rs.l *= alpha;
      rs.m = mnew;
    }
  }
  const unsigned long long sc2 = pack_f2(sc, sc), nm2 = pack_f2(-rs.m, -rs.m);
  unsigned long long ls2[2] = {0ull, 0ull};
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t v[32];
    tmem_ld32(tS_lane + c * 32, v);
    tmem_wait_ld();
    if (MASK) {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (c * 32 + j >= valid) v[j] = 0xff800000u;
    }
    uint32_t pk[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float y0, y1, p0, p1;
      unpack_f2(fma_f2(pack_f2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1])), sc2, nm2), y0, y1);
      if (!MASK && j % kFmaPairEvery == kFmaPairEvery - 1) {
        exp2_fma2(y0, y1, p0, p1);
      } else {
        p0 = ex2_approx(y0);
        p1 = ex2_approx(y1);
      }
      ls2[j & 1] = add_f2(ls2[j & 1], pack_f2(p0, p1));
      pk[j] = pack_bf2(p0, p1);
    }
    tmem_st16(tS_lane + c * 16, pk);
    if (c == 1) halfway();
  }
  float s0, s1, s2, s3;
  unpack_f2(ls2[0], s0, s1);
  unpack_f2(ls2[1], s2, s3);
  rs.l += (s0 + s1) + (s2 + s3);
}

constexpr int A2_COPY_WARPS = 6;
constexpr int A2_THREADS = (10 + A2_COPY_WARPS) * 32;   // 8 softmax warps, the MMA warp, an idle warp, the copy warps
constexpr int A2_SLOT = 2 * AT_TILE;                      // K tile, V tile
constexpr int A2_OFF_SLOT = 2 * AT_TILE;                  // after the two Q tiles
constexpr int A2_OFF_MISC = A2_OFF_SLOT + 2 * A2_SLOT;
constexpr int A2_RUN_INTS = 2 * MAX_RUNS + 8;                // one run list: starts, positions
constexpr int A2_SMEM_INTS = 2 * A2_RUN_INTS + 32;
constexpr int A2_SMEM = A2_OFF_MISC + 256 + A2_SMEM_INTS * 4 + 1024;
enum { B_S = 0, B_O = 2, B_P = 4, B_FULLK = 8, B_FULLV = 10, B_FREEK = 12, B_FREEV = 14, B_FULLQ = 16, B_COUNT = 18 };   // P: [group][half]

__global__ void __launch_bounds__(A2_THREADS, 1) attn2_kernel(
    const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ KVMaps maps,
    const uint32_t* __restrict__ ub, const int* __restrict__ qperm,
    __nv_bfloat16* __restrict__ attn_out, float* __restrict__ attn_lse, int* __restrict__ plan, int H, int N, int CQ,
    int q_row_step, int q_head_step, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + A2_OFF_MISC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + A2_OFF_MISC + B_COUNT * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + A2_OFF_MISC + B_COUNT * 8 + 8);
  int* sInt = reinterpret_cast<int*>(sm + A2_OFF_MISC + 256);
  int* sRuns = sInt;                              // two run lists (this task's, the next one's): [MAX_RUNS] starts, [MAX_RUNS + 1] positions
  int* sMisc = sInt + 2 * A2_RUN_INTS;            // [2..7] the next task: index, head, cluster, first row, rows, union length; [8], [9] runs of the two lists

  const PlanView pv = plan_view(plan, H, N, CQ);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grp = (warp >> 2) & 1, gt = tid & 127, gw = warp & 3;   // softmax warps: group, thread, warp in group

  // the kernel launched behind this one (tasks of at most QT rows) does not depend on it: let it be scheduled
  // as soon as SMs free up
  asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < B_COUNT; ++i)
      mbar_init(bars + i, (i >= B_P && i < B_P + 4) ? 4 : 1);
    mbar_init_fence();
    // all ring slots start empty: complete phase 0 of the free barriers
    for (int i = B_FREEK; i < B_FREEV + 2; ++i) mbar_arrive(bars + i);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  uint32_t tiles_done = 0, qcnt = 0;      // tiles / non-empty tasks this CTA has processed; every role counts alike
  uint32_t phS = 0, phO = 0;              // softmax warps: phases of their group's S and O barriers
  const int numTasks = pv.counters[0];
  const float sc = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
  constexpr uint32_t idescQK = make_idesc_bf16(128, KT, false, false);
  constexpr uint32_t idescPV = make_idesc_bf16(128, kD, false, true);

  // The next task of more than QT rows is prepared while the current one runs, by warp 9, which has nothing
  // else to do: cursor, task record and union length (three dependent trips to global memory), then the run
  // list of its union into the list the current task does not use.
  auto prepare_task = [&](int list) {
    int i = 0, th = 0, tc = 0, len = 0;
    if (lane == 0) {
      do { i = atomicAdd(&pv.counters[4], 1); } while (i < numTasks && pv.tasks[i].w <= QT);
      int4 tk = make_int4(0, 0, 0, 0);
      if (i < numTasks) {
        tk = pv.tasks[i];
        len = pv.kv_lens[(size_t)tk.x * CQ + tk.y];
      }
      th = tk.x;
      tc = tk.y;
      sMisc[2] = i; sMisc[3] = tk.x; sMisc[4] = tk.y; sMisc[5] = tk.z; sMisc[6] = tk.w; sMisc[7] = len;
    }
    i = __shfl_sync(0xffffffffu, i, 0);
    th = __shfl_sync(0xffffffffu, th, 0);
    tc = __shfl_sync(0xffffffffu, tc, 0);
    len = __shfl_sync(0xffffffffu, len, 0);
    if (i < numTasks && len > 0)
      build_runs_warp(pv.k_off + (size_t)th * (kC + 1), ub + ((size_t)th * CQ + tc) * (kC / 32),
                      pv.nonempty + (size_t)th * (kC / 32), sRuns + list * A2_RUN_INTS,
                      sRuns + list * A2_RUN_INTS + MAX_RUNS, sMisc + 8 + list, abort_flag, status);
  };
  int list = 0;      // the run list of the current task
  if (warp == 9) prepare_task(0);

  while (true) {
    __syncthreads();
    const int ti = sMisc[2], h = sMisc[3], qs = sMisc[5], qrows = sMisc[6], kvlen = sMisc[7];
    __syncthreads();      // everyone has the task: the record may be overwritten
    if (ti >= numTasks || *abort_flag) break;
    const size_t rowbase = (size_t)h * N + qs;
    const int* sRunStart = sRuns + list * A2_RUN_INTS;
    const int* sRunCum = sRunStart + MAX_RUNS;
    const int nruns = sMisc[8 + list];
    list ^= 1;
    if (warp == 9) prepare_task(list);

    if (kvlen == 0) {   // empty union: O = 0, lse = -inf
      for (int i = tid; i < qrows * 16; i += A2_THREADS)
        reinterpret_cast<uint4*>(attn_out + (rowbase + (i >> 4)) * kD)[i & 15] = make_uint4(0u, 0u, 0u, 0u);
      for (int r = tid; r < qrows; r += A2_THREADS) attn_lse[rowbase + r] = -INFINITY;
      continue;
    }

    const int rows0 = (qrows + 1) >> 1;                       // rows of group 0; group 1 takes the rest
    if (warp >= 10 && warp < 14) {      // the Q tiles need no run list: their gathers go first
      const int kind = (warp - 10) >> 1, oblk = (warp - 10) & 1, orow = lane * 4;
      const int off = kind ? rows0 : 0, nr = kind ? qrows - rows0 : rows0;
      int r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)      // slots past the group repeat its first row
        r[j] = h * q_head_step + qperm[rowbase + off + (orow + j < nr ? orow + j : 0)] * q_row_step;
      if (oblk == 0 && lane == 0) mbar_arrive_expect_tx(bars + B_FULLQ + kind, AT_TILE);
      tma_gather4(base + kind * AT_TILE + oblk * (KT * 128) + orow * 128, &mapQ, oblk * 64, r[0], r[1], r[2], r[3],
                  bars + B_FULLQ + kind);
    }
    const int ntiles = cdiv(kvlen, KT);
    const uint32_t g0 = tiles_done;

    if (warp >= 10 && warp < 14) {
      // ================= copy warps: the K / V stream ===============
      // warp 10, 11: the two 64-column blocks of the K tiles (above: of group 0's Q tile); warps 12, 13: those
      // of the V tiles (of group 1's Q tile).  A lane owns rows 4 lane .. 4 lane + 3 of a tile.
      const int kind = (warp - 10) >> 1, oblk = (warp - 10) & 1, orow = lane * 4;
      const bool announces = oblk == 0 && lane == 0;
      const CUtensorMap* map1 = kind ? &maps.v1 : &maps.k1;
      const CUtensorMap* map32 = kind ? &maps.v32 : &maps.k32;
      const CUtensorMap* map64 = kind ? &maps.v64 : &maps.k64;
      int cursor = 0;
      for (int t = 0; t < ntiles; ++t) {
        const uint32_t g = g0 + t, slot = g & 1u, par = (g >> 1) & 1u;
        int r[4];
        const bool whole = union_rows(sRunStart, sRunCum, nruns, kvlen, t * KT + orow, h * N, cursor, r);
        const int what = fetch_plan(r, whole, lane);
        if (!mbar_wait(bars + (kind ? B_FREEV : B_FREEK) + slot, par, abort_flag)) break;
        uint64_t* full = bars + (kind ? B_FULLV : B_FULLK) + slot;
        if (announces) mbar_arrive_expect_tx(full, AT_TILE);
        fetch_issue(what, base + A2_OFF_SLOT + slot * A2_SLOT + kind * AT_TILE + oblk * (KT * 128), map1, map32, map64,
                    oblk * 64, r, lane, full);
      }
    } else if (warp == 8) {
      // ================= MMA warp: one lane issues everything, group 0 then group 1 ===============
      // The lane is the busiest resource of the kernel (an MMA of this shape occupies the tensor pipe
      // for ~90 cycles and the issue blocks for as long), so it waits for the tiles, which land early,
      // before it waits for a group's P, and then issues P V and the next Q K^T back to back.
      if (lane == 0) {
        bool ok = true;
        // descriptor low words of the tiles (the K steps add constants to them), one high word for all
        constexpr uint32_t dhi = sdesc_hi(1024);
        const uint32_t qlo[2] = {sdesc_lo(base, 16), sdesc_lo(base + AT_TILE, 16)};
        const uint32_t klo[2] = {sdesc_lo(base + A2_OFF_SLOT, 16), sdesc_lo(base + A2_OFF_SLOT + A2_SLOT, 16)};
        const uint32_t vlo[2] = {sdesc_lo(base + A2_OFF_SLOT + AT_TILE, KT * 128),
                                 sdesc_lo(base + A2_OFF_SLOT + A2_SLOT + AT_TILE, KT * 128)};
        auto mma_qk = [&](int g, uint32_t slot) {      // S_g = Q_g K^T for the K tile in ring slot `slot`
          const uint32_t a0 = qlo[g], b0 = slot ? klo[1] : klo[0];
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            constexpr uint32_t blk = (QT * 128) >> 4;      // second 64-column block of a tile
            const uint32_t off = (s >> 2) * blk + (s & 3) * 2;
            umma_ss_lo(tmem + g * 256, a0 + off, b0 + off, dhi, idescQK, s > 0 ? 1u : 0u);
          }
          umma_commit(bars + B_S + g);
          if (g == 1) umma_commit(bars + B_FREEK + slot);      // covers group 0's MMAs too: same issuer, in order
        };
        tc_fence_after();
        ok = mbar_wait(bars + B_FULLQ + 0, qcnt & 1u, abort_flag) && mbar_wait(bars + B_FULLQ + 1, qcnt & 1u, abort_flag) &&
             mbar_wait(bars + B_FULLK + (g0 & 1u), (g0 >> 1) & 1u, abort_flag);
        if (ok) {
          tc_fence_after();
          mma_qk(0, g0 & 1u);
          mma_qk(1, g0 & 1u);
        }
        for (int t = 0; t < ntiles && ok; ++t) {
          const uint32_t tg = g0 + t, slot = tg & 1u;
          const bool more = t + 1 < ntiles;
          const uint32_t v0 = slot ? vlo[1] : vlo[0];
          if (!mbar_wait(bars + B_FULLV + slot, (tg >> 1) & 1u, abort_flag)) break;
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            const uint32_t tS = tmem + g * 256, tO = tS + 128;
            // P_g reaches tensor memory in two halves of 64 keys; every P barrier completes once per tile
            if (!mbar_wait(bars + B_P + g * 2, tg & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int s8 = 0; s8 < 4; ++s8)
              umma_ts_lo(tO, tS + s8 * 8, v0 + s8 * (2048 >> 4), dhi, idescPV, (t > 0 || s8 > 0) ? 1u : 0u);
            if (!mbar_wait(bars + B_P + g * 2 + 1, tg & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
#pragma unroll
            for (int s8 = 4; s8 < 8; ++s8)
              umma_ts_lo(tO, tS + s8 * 8, v0 + s8 * (2048 >> 4), dhi, idescPV, 1u);
            umma_commit(bars + B_O + g);
            if (g == 1) umma_commit(bars + B_FREEV + slot);
            if (more) {
              if (g == 0) {      // the next K tile is first needed here
                if (!mbar_wait(bars + B_FULLK + (slot ^ 1u), ((tg + 1) >> 1) & 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
              }
              mma_qk(g, slot ^ 1u);
            }
          }
        }
      }
    } else if (warp < 8) {
      // ================= softmax warps: 128 threads per group, one query row each =================
      const int myoff = grp ? rows0 : 0, myrows = grp ? qrows - rows0 : rows0;
      const bool warp_has_rows = gw * 32 < myrows;
      const uint32_t tS = tmem + grp * 256, tO = tS + 128;
      const uint32_t tS_lane = tmem_addr(tS, gw * 32, 0), tO_lane = tmem_addr(tO, gw * 32, 0);
      uint64_t* barS = bars + B_S + grp;
      uint64_t* barO = bars + B_O + grp;
      RowState rs;
      rs.m = -INFINITY;
      rs.l = 0.f;
      bool dead = false;
      for (int t = 0; t < ntiles; ++t) {
        if (!mbar_wait(barS, phS, abort_flag)) { dead = true; break; }
        phS ^= 1u;
        if (t > 0) {      // P V of tile t - 1 finished before Q K^T of tile t: this only tracks the phase
          if (!mbar_wait(barO, phO, abort_flag)) { dead = true; break; }
          phO ^= 1u;
        }
        tc_fence_after();
        // A warp whose rows all lie past the group's last row skips the arithmetic: its P rows stay
        // whatever S held, which only reaches O rows that are never stored.
        auto halfway = [&]() {      // keys 0 .. 63 of P are in tensor memory
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + B_P + grp * 2);
        };
        if (warp_has_rows) {
          const int valid = kvlen - t * KT;
          if (valid >= KT) softmax_tile<false>(tS_lane, tO_lane, rs, KT, t == 0, sc, halfway);
          else softmax_tile<true>(tS_lane, tO_lane, rs, valid, t == 0, sc, halfway);
          tmem_wait_st();
        } else {
          halfway();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + B_P + grp * 2 + 1);
      }
      if (!dead) {
        if (!mbar_wait(barO, phO, abort_flag)) dead = true;
        else phO ^= 1u;
      }
      if (!dead) {
        tc_fence_after();
        if (warp_has_rows) {
          const float inv = 1.0f / rs.l;
          const bool wr = gt < myrows;
          uint4* dst = reinterpret_cast<uint4*>(attn_out + (rowbase + myoff + gt) * kD);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(tO_lane + c * 32, v);
            tmem_wait_ld();
            if (wr) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                uint4 o;
                o.x = pack_bf2(__uint_as_float(v[8 * g + 0]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
                o.y = pack_bf2(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
                o.z = pack_bf2(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
                o.w = pack_bf2(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
                dst[c * 4 + g] = o;
              }
            }
          }
          if (wr) attn_lse[rowbase + myoff + gt] = (rs.m + log2f(rs.l)) * 0.6931471805599453f;
        }
        tc_fence_before();
      }
    }
    tiles_done += ntiles;
    ++qcnt;
  }
  if (*abort_flag) {
    if (tid == 0 && status) atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
    // a wait gave up: let tile copies still in flight land before the shared memory is released
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
// exact attention, tasks of at most QT rows
// ---------------------------------------------------------------------------
// The same roles as attn2_kernel with one row group and single K, V and Q buffers, two CTAs to an SM
// (256 tensor-memory columns and 110 KB of shared memory each) so that one CTA's softmax runs under the
// other's loads and products:
//   warps 0..3   softmax, one thread per query row
//   warp 4       one lane issues every MMA
//   warps 5..7   the K and V tiles (and the task's Q tile) by TMA (see fetch_plan).  A TMA instruction holds
//                its warp for about 70 cycles per lane, which threads that also compute cannot afford, and
//                one warp alone would need longer for a K tile than the softmax takes.
// Fill g of the K (V) buffer, g counting the tiles this CTA has processed, waits for phase g of freeK (freeV) -
// phase 0 is completed at start-up, phase g by the commit behind the product that read fill g - 1 - and
// completes phase g of fullK (fullV).
constexpr int A1_THREADS = 8 * 32;
constexpr int A1_OFF_MISC = 3 * AT_TILE;                  // Q, K, V tiles
constexpr int A1_SMEM_INTS = 2 * MAX_RUNS + 8 + 32;
constexpr int A1_SMEM = A1_OFF_MISC + 256 + A1_SMEM_INTS * 4 + 1024;
enum { C_S = 0, C_O = 1, C_P = 2, C_FULLK = 4, C_FULLV, C_FREEK, C_FREEV, C_FULLQ, C_COUNT };      // P: [half]
static_assert(2 * (A1_SMEM + 1024) <= 228 * 1024, "two CTAs share an SM");

__global__ void __launch_bounds__(A1_THREADS, 2) attn_kernel(
    const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ KVMaps maps,
    const uint32_t* __restrict__ ub, const int* __restrict__ qperm,
    __nv_bfloat16* __restrict__ attn_out, float* __restrict__ attn_lse, int* __restrict__ plan, int H, int N, int CQ,
    int q_row_step, int q_head_step, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sQ = base, sK = base + AT_TILE, sV = base + 2 * AT_TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + A1_OFF_MISC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + A1_OFF_MISC + C_COUNT * 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + A1_OFF_MISC + C_COUNT * 8 + 8);
  int* sInt = reinterpret_cast<int*>(sm + A1_OFF_MISC + 256);
  int* sRunStart = sInt;                          // [MAX_RUNS]
  int* sRunCum = sRunStart + MAX_RUNS;            // [MAX_RUNS + 1]
  int* sMisc = sRunCum + MAX_RUNS + 8;            // [1] runs; [2..7] the next task: index, head, cluster, first row, rows, union length

  const PlanView pv = plan_view(plan, H, N, CQ);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    *abort_flag = 0;
    for (int i = 0; i < C_COUNT; ++i)
      mbar_init(bars + i, (i == C_P || i == C_P + 1) ? 4 : ((i == C_FULLK || i == C_FULLV) ? 3 : 1));
    mbar_init_fence();
    mbar_arrive(bars + C_FREEK);      // both buffers start empty
    mbar_arrive(bars + C_FREEV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 128;
  uint32_t tiles_done = 0, qcnt = 0;      // tiles / non-empty tasks this CTA has processed; every role counts alike
  uint32_t phS = 0, phO = 0;              // softmax warps: phases of the S and O barriers
  const int numTasks = pv.counters[0];
  const float sc = 0.08838834764831845f * 1.4426950408889634f;   // 1/sqrt(128) * log2(e)
  constexpr uint32_t idescQK = make_idesc_bf16(128, KT, false, false);
  constexpr uint32_t idescPV = make_idesc_bf16(128, kD, false, true);

  // The next task of at most QT rows (the two-tile kernel takes the others) is fetched - cursor, task record,
  // union length: three dependent trips to global memory - by a copy warp once it has issued the current
  // task's last tile, while the other roles are still busy with it.
  auto fetch_task = [&]() {
    int i;
    do { i = atomicAdd(&pv.counters[1], 1); } while (i < numTasks && pv.tasks[i].w > QT);
    int4 tk = make_int4(0, 0, 0, 0);
    int len = 0;
    if (i < numTasks) {
      tk = pv.tasks[i];
      len = pv.kv_lens[(size_t)tk.x * CQ + tk.y];
    }
    sMisc[2] = i; sMisc[3] = tk.x; sMisc[4] = tk.y; sMisc[5] = tk.z; sMisc[6] = tk.w; sMisc[7] = len;
  };
  if (warp == 7 && lane == 0) fetch_task();

  while (true) {
    __syncthreads();
    const int ti = sMisc[2], h = sMisc[3], qc = sMisc[4], qs = sMisc[5], qrows = sMisc[6], kvlen = sMisc[7];
    __syncthreads();      // everyone has the task: the record may be overwritten
    if (ti >= numTasks || *abort_flag) break;
    const size_t rowbase = (size_t)h * N + qs;

    if (kvlen == 0) {   // empty union: O = 0, lse = -inf
      if (warp == 7 && lane == 0) fetch_task();
      for (int i = tid; i < qrows * 16; i += A1_THREADS)
        reinterpret_cast<uint4*>(attn_out + (rowbase + (i >> 4)) * kD)[i & 15] = make_uint4(0u, 0u, 0u, 0u);
      for (int r = tid; r < qrows; r += A1_THREADS) attn_lse[rowbase + r] = -INFINITY;
      continue;
    }
    if (warp == 5) {      // the task's Q tile needs no run list: its gathers go first; slots past the task repeat its first row
      const int orow = lane * 4;
      int r[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        r[j] = h * q_head_step + qperm[rowbase + (orow + j < qrows ? orow + j : 0)] * q_row_step;
      if (lane == 0) mbar_arrive_expect_tx(bars + C_FULLQ, AT_TILE);
      tma_gather4(sQ + orow * 128, &mapQ, 0, r[0], r[1], r[2], r[3], bars + C_FULLQ);
      tma_gather4(sQ + KT * 128 + orow * 128, &mapQ, 64, r[0], r[1], r[2], r[3], bars + C_FULLQ);
    }

    if (!build_runs(pv.k_off + (size_t)h * (kC + 1), ub + ((size_t)h * CQ + qc) * (kC / 32),
                    pv.nonempty + (size_t)h * (kC / 32), sRunStart, sRunCum, sMisc, abort_flag, status))
      break;
    const int nruns = sMisc[1];
    const int ntiles = cdiv(kvlen, KT);
    const uint32_t g0 = tiles_done;

    if (warp >= 5) {
      // ================= copy warps =================
      // K and V tiles hold the same rows, so one fetch plan serves both tiles and both of their 64-column
      // blocks; the three warps share its instructions (the n-th issuing lane belongs to warp n mod 3), K
      // first: the next Q K^T waits for it.
      const int cw = warp - 5, orow = lane * 4;
      int cursor = 0;
      for (int t = 0; t < ntiles; ++t) {
        const uint32_t g = g0 + t;
        int r[4];
        const bool whole = union_rows(sRunStart, sRunCum, nruns, kvlen, t * KT + orow, h * N, cursor, r);
        int what = fetch_plan(r, whole, lane);
        const unsigned issuing = __ballot_sync(0xffffffffu, what != FETCH_NONE);
        if (__popc(issuing & ((1u << lane) - 1u)) % 3 != cw) what = FETCH_NONE;
        if (!mbar_wait(bars + C_FREEK, g & 1u, abort_flag)) break;
        // every copy warp arrives on the full barrier, so that none of them can fall two phases behind the
        // free barrier it waits on (a warp may have nothing to fetch for a tile)
        if (lane == 0) { if (cw == 0) mbar_arrive_expect_tx(bars + C_FULLK, AT_TILE); else mbar_arrive(bars + C_FULLK); }
        fetch_issue(what, sK, &maps.k1, &maps.k32, &maps.k64, 0, r, lane, bars + C_FULLK);
        fetch_issue(what, sK + KT * 128, &maps.k1, &maps.k32, &maps.k64, 64, r, lane, bars + C_FULLK);
        if (!mbar_wait(bars + C_FREEV, g & 1u, abort_flag)) break;
        if (lane == 0) { if (cw == 0) mbar_arrive_expect_tx(bars + C_FULLV, AT_TILE); else mbar_arrive(bars + C_FULLV); }
        fetch_issue(what, sV, &maps.v1, &maps.v32, &maps.v64, 0, r, lane, bars + C_FULLV);
        fetch_issue(what, sV + KT * 128, &maps.v1, &maps.v32, &maps.v64, 64, r, lane, bars + C_FULLV);
      }
      if (warp == 7 && lane == 0) fetch_task();
    } else if (warp == 4) {
      // ================= MMA warp: one lane issues everything =================
      if (lane == 0) {
        constexpr uint32_t dhi = sdesc_hi(1024);
        const uint32_t qlo = sdesc_lo(sQ, 16), klo = sdesc_lo(sK, 16), vlo = sdesc_lo(sV, KT * 128);
        auto mma_qk = [&]() {      // S = Q K^T; its completion also frees the K buffer
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            constexpr uint32_t blk = (QT * 128) >> 4;      // second 64-column block of a tile
            const uint32_t off = (s >> 2) * blk + (s & 3) * 2;
            umma_ss_lo(tS, qlo + off, klo + off, dhi, idescQK, s > 0 ? 1u : 0u);
          }
          umma_commit(bars + C_S);
          umma_commit(bars + C_FREEK);
        };
        tc_fence_after();
        bool ok = mbar_wait(bars + C_FULLQ, qcnt & 1u, abort_flag) && mbar_wait(bars + C_FULLK, g0 & 1u, abort_flag);
        if (ok) {
          tc_fence_after();
          mma_qk();
        }
        for (int t = 0; t < ntiles && ok; ++t) {
          const uint32_t tg = g0 + t;
          const bool more = t + 1 < ntiles;
          if (!mbar_wait(bars + C_FULLV, tg & 1u, abort_flag)) break;
          // P reaches tensor memory in two halves of 64 keys; both P barriers complete once per tile
          if (!mbar_wait(bars + C_P, tg & 1u, abort_flag)) break;
          tc_fence_after();
#pragma unroll
          for (int s8 = 0; s8 < 4; ++s8)
            umma_ts_lo(tO, tS + s8 * 8, vlo + s8 * (2048 >> 4), dhi, idescPV, (t > 0 || s8 > 0) ? 1u : 0u);
          if (!mbar_wait(bars + C_P + 1, tg & 1u, abort_flag)) break;
          tc_fence_after();
#pragma unroll
          for (int s8 = 4; s8 < 8; ++s8)
            umma_ts_lo(tO, tS + s8 * 8, vlo + s8 * (2048 >> 4), dhi, idescPV, 1u);
          umma_commit(bars + C_O);
          umma_commit(bars + C_FREEV);
          if (more) {
            if (!mbar_wait(bars + C_FULLK, (tg + 1) & 1u, abort_flag)) break;
            tc_fence_after();
            mma_qk();
          }
        }
      }
    } else {
      // ================= softmax warps: one query row per thread =================
      const bool warp_has_rows = warp * 32 < qrows;
      const uint32_t tS_lane = tmem_addr(tS, warp * 32, 0), tO_lane = tmem_addr(tO, warp * 32, 0);
      RowState rs;
      rs.m = -INFINITY;
      rs.l = 0.f;
      bool dead = false;
      for (int t = 0; t < ntiles; ++t) {
        if (!mbar_wait(bars + C_S, phS, abort_flag)) { dead = true; break; }
        phS ^= 1u;
        if (t > 0) {      // P V of tile t - 1 finished before Q K^T of tile t: this only tracks the phase
          if (!mbar_wait(bars + C_O, phO, abort_flag)) { dead = true; break; }
          phO ^= 1u;
        }
        tc_fence_after();
        // A warp whose rows all lie past the task's last row skips the arithmetic: its P rows stay whatever S
        // held, which only reaches O rows that are never stored.
        auto halfway = [&]() {      // keys 0 .. 63 of P are in tensor memory
          tmem_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + C_P);
        };
        if (warp_has_rows) {
          const int valid = kvlen - t * KT;
          if (valid >= KT) softmax_tile<false>(tS_lane, tO_lane, rs, KT, t == 0, sc, halfway);
          else softmax_tile<true>(tS_lane, tO_lane, rs, valid, t == 0, sc, halfway);
          tmem_wait_st();
        } else {
          halfway();
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bars + C_P + 1);
      }
      if (!dead) {
        if (!mbar_wait(bars + C_O, phO, abort_flag)) dead = true;
        else phO ^= 1u;
      }
      if (!dead) {
        tc_fence_after();
        if (warp_has_rows) {
          const float inv = 1.0f / rs.l;
          const bool wr = tid < qrows;
          uint4* dst = reinterpret_cast<uint4*>(attn_out + (rowbase + tid) * kD);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t v[32];
            tmem_ld32(tO_lane + c * 32, v);
            tmem_wait_ld();
            if (wr) {
#pragma unroll
              for (int g = 0; g < 4; ++g) {
                uint4 o;
                o.x = pack_bf2(__uint_as_float(v[8 * g + 0]) * inv, __uint_as_float(v[8 * g + 1]) * inv);
                o.y = pack_bf2(__uint_as_float(v[8 * g + 2]) * inv, __uint_as_float(v[8 * g + 3]) * inv);
                o.z = pack_bf2(__uint_as_float(v[8 * g + 4]) * inv, __uint_as_float(v[8 * g + 5]) * inv);
                o.w = pack_bf2(__uint_as_float(v[8 * g + 6]) * inv, __uint_as_float(v[8 * g + 7]) * inv);
                dst[c * 4 + g] = o;
              }
            }
          }
          if (wr) attn_lse[rowbase + tid] = (rs.m + log2f(rs.l)) * 0.6931471805599453f;
        }
        tc_fence_before();
      }
    }
    tiles_done += ntiles;
    ++qcnt;
  }
  if (*abort_flag) {
    if (tid == 0 && status) atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
    // a wait gave up: let tile copies still in flight land before the shared memory is released
    for (int i = 0; i < 100; ++i) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
  // This kernel may have started while the kernel launched before it (the tasks above QT rows) was still
  // running.  No CTA leaves before that grid has completed and its results are visible, so that this grid's
  // completion, which later work in the stream waits for, implies the other's.  (Without a programmatic
  // launch the instruction returns at once.)
  asm volatile("griddepcontrol.wait;\n" ::: "memory");
}

// ---------------------------------------------------------------------------
// centroid residual + merge, 128 sorted queries per CTA
// ---------------------------------------------------------------------------
constexpr int TL_Q = 128;                 // sorted queries per CTA (one softmax thread per row)
constexpr int TL_H = 64;                  // centroids per step
constexpr int TL_NH = kC / TL_H;          // steps per CTA
constexpr int TL_STAGES = 3;              // ring depth of the centroid and value-sum tiles
constexpr int TL_SQ = TL_Q * 128;         // 16 KB: QU rows padded to 128 B
constexpr int TL_SC = TL_H * 128;         // 8 KB per stage: cks rows padded to 128 B
constexpr int TL_SV = TL_H * kD * 2;      // 16 KB per stage
constexpr int TL_OFF_C = TL_SQ;
constexpr int TL_OFF_V = TL_OFF_C + TL_STAGES * TL_SC;
constexpr int TL_OFF_CNT = TL_OFF_V + TL_STAGES * TL_SV;
constexpr int TL_OFF_BAR = TL_OFF_CNT + kC * 4;
// 97 KB: two CTAs share an SM, and no more than two (tensor memory holds two 256-column allocations)
constexpr int TL_SMEM = TL_OFF_BAR + 128 + 1024;
constexpr int TL_THREADS = 160;           // warps 0..3: one softmax thread per row; warp 4: the MMA lane
static_assert(TL_NH % 2 == 0 && TL_NH >= 4, "the two score regions alternate");
static_assert(3 * TL_SMEM > 227 * 1024, "at most two CTAs may share an SM");

// Work is pipelined over steps of 64 centroids.  Tensor memory holds two 64-column score regions and the
// 128-column accumulator T.  For step i (region b = i & 1):
//   MMA lane      S_b = QU cks_i^T  ->  commit on sReady[b]
//   softmax rows  wait sReady[b]; p = exp2(S_b - m) masked by the row's union, packed to bf16 into S_b;
//                 arrive on pReady[b]
//   MMA lane      wait pReady[b]; T += P_b sumv_i; S_b = QU cks_{i+2}^T; commit on sReady[b]
// so the tensor work of one region runs under the softmax of the other.  Two rings feed the products.  The
// softmax threads issue the cp.async copies of cks_{i+3} at the start of step i, into the stage that
// sReady[b] has just declared free, and before arriving on pReady[b] they wait for the copy issued one step
// earlier (cks_{i+2}), which the MMA lane is about to read.  The MMA lane itself fetches sumv_{i+1} with two
// TMA tile loads once pReady[b] of step i shows that every row has seen the commit behind the product of
// step i - 2, and waits for sumv_i on the stage's byte-counting barrier before T += P_b sumv_i.
__global__ void __launch_bounds__(TL_THREADS, 2) tail_kernel(
    const __grid_constant__ CUtensorMap mapSumv, const __nv_bfloat16* __restrict__ attn_out,
    const float* __restrict__ attn_lse,
    const __nv_bfloat16* __restrict__ QU, const __nv_bfloat16* __restrict__ cks,
    const int* __restrict__ ksz, const uint32_t* __restrict__ ub,
    const int* __restrict__ qlab, const int* __restrict__ qperm, const float* __restrict__ lam_s,
    const float* __restrict__ tailw_ptr, __nv_bfloat16* __restrict__ out, long long out_row_stride,
    long long out_head_stride, int N, int CQ,
    int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sQ = base, sC = base + TL_OFF_C, sV = base + TL_OFF_V;
  float* sCnt = reinterpret_cast<float*>(sm + TL_OFF_CNT);
  uint64_t* sReady = reinterpret_cast<uint64_t*>(sm + TL_OFF_BAR);        // [2], one arrival (tcgen05.commit)
  uint64_t* pReady = sReady + 2;                                          // [2], 128 arrivals
  uint64_t* vFull = sReady + 4;                                           // [TL_STAGES], bytes of one value-sum tile
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + TL_OFF_BAR + 64);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + TL_OFF_BAR + 80);

  const int tid = threadIdx.x, warp = tid >> 5;
  const bool soft = warp < 4;
  const int h = blockIdx.y, qs = blockIdx.x * TL_Q;
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  if (tid == 0) {
    *abort_flag = 0;
    mbar_init(sReady + 0, 1);
    mbar_init(sReady + 1, 1);
    mbar_init(pReady + 0, TL_Q);
    mbar_init(pReady + 1, TL_Q);
    for (int st = 0; st < TL_STAGES; ++st) mbar_init(vFull + st, 1);
    mbar_init_fence();
  }
  const int j = qs + tid;
  const bool active = soft && j < N;
  const int orig = active ? qperm[(size_t)h * N + j] : 0;
  const int label = active ? qlab[(size_t)h * N + orig] : 0;
  const uint32_t* mrow = ub + ((size_t)h * CQ + label) * (kC / 32);

  auto load_c = [&](int step) {   // centroid rows of one step: 64 rows x 64 B into 128-byte rows
    const int ch = tid & 3, r0 = tid >> 2;
    const __nv_bfloat16* src = cks + ((size_t)h * kC + step * TL_H) * kR + ch * 8;
    const uint32_t dst = sC + (step % TL_STAGES) * TL_SC;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int r = r0 + 32 * u;
      cp_async16(dst + sw128(r, ch), src + (size_t)r * kR, 16u);
    }
  };
  if (soft) {
    // group 0: the copies that depend on nothing (centroids of steps 0..2) go first
    load_c(0);
    load_c(1);
    load_c(2);
    cp_async_commit();
    // group 1: QU rows of the 128 sorted queries (64 B each, 4 chunks), behind the loads of their indices
    const int ch = tid & 3, r0 = tid >> 2;
    int o4[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) o4[u] = qs + r0 + 32 * u < N ? qperm[(size_t)h * N + qs + r0 + 32 * u] : -1;
    const int4* ksz4 = reinterpret_cast<const int4*>(ksz + (size_t)h * kC);
    int4 kz[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) kz[u] = ksz4[tid + TL_Q * u];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int r = r0 + 32 * u;
      cp_async16(sQ + sw128(r, ch), QU + ((size_t)h * N + max(o4[u], 0)) * kR + ch * 8, o4[u] >= 0 ? 16u : 0u);
    }
    cp_async_commit();
#pragma unroll
    for (int u = 0; u < 4; ++u)
      reinterpret_cast<float4*>(sCnt)[tid + TL_Q * u] =
          make_float4((float)kz[u].x, (float)kz[u].y, (float)kz[u].z, (float)kz[u].w);
    cp_async_wait<0>();
    fence_proxy_async();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS = tmem, tO = tmem + 2 * TL_H;
  constexpr uint32_t idescS = make_idesc_bf16(128, TL_H, false, false);
  constexpr uint32_t idescT = make_idesc_bf16(128, kD, false, true);
  constexpr float LOG2E = 1.4426950408889634f;

  auto issue_scores = [&](int step) {   // S_(step & 1) = QU cks_step^T, K = 32
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const uint64_t ad = make_sdesc(sQ + s * 32, 16, 1024);
      const uint64_t bd = make_sdesc(sC + (step % TL_STAGES) * TL_SC + s * 32, 16, 1024);
      umma_ss(tS + (step & 1) * TL_H, ad, bd, idescS, s > 0 ? 1u : 0u);
    }
  };

  // value sums of one step: 64 rows x 256 B as two 64-column blocks, one TMA tile load each
  auto load_v = [&](int step) {
    uint64_t* bar = vFull + step % TL_STAGES;
    const uint32_t dst = sV + (step % TL_STAGES) * TL_SV;
    mbar_arrive_expect_tx(bar, TL_SV);
    tma_load_tile(dst, &mapSumv, 0, h * kC + step * TL_H, bar);
    tma_load_tile(dst + TL_H * 128, &mapSumv, 64, h * kC + step * TL_H, bar);
  };
  if (tid == TL_Q) {
    // ---- MMA lane ----
    load_v(0);
    issue_scores(0);
    umma_commit(sReady + 0);
    issue_scores(1);
    umma_commit(sReady + 1);
    for (int i = 0; i < TL_NH; ++i) {
      const int b = i & 1;
      if (!mbar_wait(pReady + b, (i >> 1) & 1, abort_flag)) break;
      tc_fence_after();
      // every softmax thread has seen the commit behind the product of step i - 2: its stage is free
      if (i + 1 < TL_NH) load_v(i + 1);
      if (!mbar_wait(vFull + i % TL_STAGES, (i / TL_STAGES) & 1, abort_flag)) break;
      const uint32_t vb = sV + (i % TL_STAGES) * TL_SV;
#pragma unroll
      for (int s8 = 0; s8 < TL_H / 16; ++s8) {
        const uint64_t bd = make_sdesc(vb + s8 * 2048, TL_H * 128, 1024);
        umma_ts(tO, tS + b * TL_H + s8 * 8, bd, idescT, (i > 0 || s8 > 0) ? 1u : 0u);
      }
      if (i + 2 < TL_NH) issue_scores(i + 2);
      umma_commit(sReady + b);
    }
  }
  bool dead = false;
  if (soft) {
    // ---- softmax rows ----
    const uint32_t tS_lane = tmem_addr(tS, warp * 32, 0), tO_lane = tmem_addr(tO, warp * 32, 0);
    float m = -INFINITY, phi = 0.f;     // m in log2 units
    uint2 mw_next = *reinterpret_cast<const uint2*>(mrow);   // union bits of the step's 64 centroids
    for (int i = 0; i < TL_NH; ++i) {
      const int b = i & 1;
      if (!mbar_wait(sReady + b, (i >> 1) & 1, abort_flag)) { dead = true; break; }
      tc_fence_after();
      // the stage of cks_i is free now
      if (i + 3 < TL_NH) load_c(i + 3);
      cp_async_commit();
      const uint2 mw2 = mw_next;
      if (i + 1 < TL_NH) mw_next = *reinterpret_cast<const uint2*>(mrow + (i + 1) * 2);
      float s[TL_H];
#pragma unroll
      for (int c = 0; c < TL_H / 32; ++c) {
        uint32_t v[32];
        tmem_ld32(tS_lane + b * TL_H + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int k = 0; k < 32; ++k) s[c * 32 + k] = __uint_as_float(v[k]);
      }
      // The scores are rounded to fp16 exactly as the selection saw them, and the members of the row's union
      // become -inf, both on packed pairs: shifting a word of union bits left by 7 - r puts the bits of the
      // centroids r, r + 8, r + 16, r + 24 on the sign bits of its four bytes, and a byte permute with sign
      // replication turns two such bytes into the select mask of a pair.  The scores stay in natural-log
      // units here; log2(e) is folded into the exponent's multiply-add below.
      const uint32_t mw[2] = {mw2.x, mw2.y};
      uint32_t sh[2][8];
#pragma unroll
      for (int w = 0; w < 2; ++w)
#pragma unroll
        for (int r = 0; r < 8; ++r) sh[w][r] = mw[w] << (7 - r);
      __half2 hm[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) hm[a] = __float2half2_rn(-INFINITY);
#pragma unroll
      for (int k = 0; k < TL_H; k += 2) {
        const int w = k >> 5, r = k & 7, jb = (k & 31) >> 3;
        const uint32_t sel = (8u | jb) * 0x11u | ((8u | (4u + jb)) * 0x11u) << 8;
        uint32_t msk;   // selector bit 3 of a nibble: replicate the chosen byte's sign over the result byte
        asm("prmt.b32 %0, %1, %2, %3;" : "=r"(msk) : "r"(sh[w][r]), "r"(sh[w][r + 1]), "r"(sel));
        const __half2 h2 = __floats2half2_rn(s[k], s[k + 1]);
        const uint32_t u = (*reinterpret_cast<const uint32_t*>(&h2) & ~msk) | (0xFC00FC00u & msk);
        const __half2 hq = *reinterpret_cast<const __half2*>(&u);
        hm[(k >> 1) & 3] = __hmax2(hm[(k >> 1) & 3], hq);
        const float2 g = __half22float2(hq);
        s[k] = g.x;
        s[k + 1] = g.y;
      }
      const float2 mxp = __half22float2(__hmax2(__hmax2(hm[0], hm[1]), __hmax2(hm[2], hm[3])));
      const float mx = fmaxf(mxp.x, mxp.y) * LOG2E;
      const bool grow = mx > m + kLazy || (m == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, grow)) {
        const float mnew = grow ? mx : m;
        const float alpha = (m == -INFINITY) ? 0.f : ex2_approx(m - mnew);
        if (i > 0) {
          // T is rescaled in place: the product of step i - 1 may still be running, its commit is the
          // next completion of the other region's barrier (the same one step i + 1 waits for)
          if (!mbar_wait(sReady + (b ^ 1), (((i - 1) >> 1) + 1) & 1, abort_flag)) { dead = true; break; }
          tc_fence_after();
          rescale_rows(tO_lane, alpha);
        }
        phi *= alpha;
        m = mnew;
      }
      const float nm = (m == -INFINITY) ? 0.f : -m;
      const unsigned long long l2e2 = pack_f2(LOG2E, LOG2E), nm2 = pack_f2(nm, nm);
      const float4* cnt4 = reinterpret_cast<const float4*>(sCnt + i * TL_H);
      float ps4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t pk[TL_H / 2];
#pragma unroll
      for (int k = 0; k < TL_H / 4; ++k) {
        const float4 cn = cnt4[k];
        float y0, y1, y2, y3, p0, p1, p2, p3;
        unpack_f2(fma_f2(pack_f2(s[4 * k], s[4 * k + 1]), l2e2, nm2), y0, y1);
        unpack_f2(fma_f2(pack_f2(s[4 * k + 2], s[4 * k + 3]), l2e2, nm2), y2, y3);
        // every third group of four on the FMA pipe: the two CTAs of an SM share one special-function unit.
        // (A member of the row's union, -inf here, then weighs 2^-125 instead of an exact zero.)
        if (k % 3 == 2) {
          exp2_fma2(y0, y1, p0, p1);
          exp2_fma2(y2, y3, p2, p3);
        } else {
          p0 = ex2_approx(y0);
          p1 = ex2_approx(y1);
          p2 = ex2_approx(y2);
          p3 = ex2_approx(y3);
        }
        ps4[k & 3] = fmaf(p1, cn.y, fmaf(p0, cn.x, ps4[k & 3]));
        ps4[(k + 2) & 3] = fmaf(p3, cn.w, fmaf(p2, cn.z, ps4[(k + 2) & 3]));
        pk[2 * k] = pack_bf2(p0, p1);
        pk[2 * k + 1] = pack_bf2(p2, p3);
      }
      phi += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
      tmem_st32(tS_lane + b * TL_H, pk);
      tmem_wait_st();
      // cks_{i+2} (issued one step ago) must have landed before the MMA lane reads it
      cp_async_wait<1>();
      fence_proxy_async();
      tc_fence_before();
      mbar_arrive(pReady + b);
    }
    // the row of the exact part is fetched while the last products finish
    const uint4* src = reinterpret_cast<const uint4*>(attn_out + ((size_t)h * N + (active ? j : 0)) * kD);
    uint4 ex16[16];
#pragma unroll
    for (int g = 0; g < 16; ++g) ex16[g] = ldg_nc_v4(src + g);
    const float lam = lam_s[h], tw = *tailw_ptr;
    const float le = active ? attn_lse[(size_t)h * N + j] : 0.f;
    // the last commit on each region's barrier covers every product
    if (!dead) dead = !mbar_wait(sReady + 0, (TL_NH >> 1) & 1, abort_flag);
    if (!dead) dead = !mbar_wait(sReady + 1, (TL_NH >> 1) & 1, abort_flag);
    tc_fence_after();
    if (!dead) {
      // merge with the exact part (natural-log units from here on); rows past N
      // only take part in the warp-collective TMEM loads
      const float mt = (m == -INFINITY) ? 0.f : m * 0.6931471805599453f;
      float ex, st;
      if (le >= mt) { ex = 1.0f; st = __expf(mt - le); } else { ex = __expf(le - mt); st = 1.0f; }
      const float ph = st * phi;
      const bool bad = ph <= 1.0e-6f * ex;
      const float inv = 1.0f / fmaxf(ex + ph * tw, 1.0e-12f);
      const float we = bad ? 1.0f : ex * inv;
      const float wt = bad ? 0.0f : st * tw * lam * inv;
      uint4* dst = reinterpret_cast<uint4*>(out + (size_t)h * out_head_stride + (size_t)orig * out_row_stride);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld32(tO_lane + c * 32, v);
        tmem_wait_ld();
        if (active) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const uint4 e = ex16[c * 4 + g];
            uint4 o;
            if (bad) {
              o = e;
            } else {
              o.x = pack_bf2(fmaf(wt, __uint_as_float(v[8 * g + 0]), we * bf_lo(e.x)), fmaf(wt, __uint_as_float(v[8 * g + 1]), we * bf_hi(e.x)));
              o.y = pack_bf2(fmaf(wt, __uint_as_float(v[8 * g + 2]), we * bf_lo(e.y)), fmaf(wt, __uint_as_float(v[8 * g + 3]), we * bf_hi(e.y)));
              o.z = pack_bf2(fmaf(wt, __uint_as_float(v[8 * g + 4]), we * bf_lo(e.z)), fmaf(wt, __uint_as_float(v[8 * g + 5]), we * bf_hi(e.z)));
              o.w = pack_bf2(fmaf(wt, __uint_as_float(v[8 * g + 6]), we * bf_lo(e.w)), fmaf(wt, __uint_as_float(v[8 * g + 7]), we * bf_hi(e.w)));
            }
            dst[c * 4 + g] = o;
          }
        }
      }
    }
    cp_async_wait<0>();
  }
  if (*abort_flag && (tid & 31) == 0 && status) atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace t2t

using namespace t2t;

namespace {
// Launch facts that do not change between calls: looked up (and the kernels' shared-memory limits raised)
// once per device and process, not on every call.
struct DeviceFacts {
  bool ready;
  int sms;
};
std::mutex g_facts_mutex;
const DeviceFacts* device_facts() {
  static DeviceFacts table[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(g_facts_mutex);
  DeviceFacts* f = &table[dev];
  if (!f->ready) {
    int sms = 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return nullptr;
    if (cudaFuncSetAttribute(attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A1_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(attn2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, A2_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TL_SMEM) != cudaSuccess)
      return nullptr;
    f->sms = sms;
    f->ready = true;
  }
  return f;
}

// Tensor maps are pure functions of (base address, rows, box rows): the operator passes the same few buffers on
// every call, so the last encodings are kept.
struct MapSlot {
  const void* base;
  uint64_t rows;
  uint32_t box_rows;
  CUtensorMap map;
};
std::mutex g_map_mutex;
bool cached_row_map(CUtensorMap* out, const void* base, uint64_t rows, uint32_t box_rows) {
  static MapSlot slots[32] = {};
  static unsigned next = 0;
  std::lock_guard<std::mutex> lock(g_map_mutex);
  for (const MapSlot& s : slots)
    if (s.base == base && s.rows == rows && s.box_rows == box_rows && s.base != nullptr) { *out = s.map; return true; }
  MapSlot fresh;
  fresh.base = base;
  fresh.rows = rows;
  fresh.box_rows = box_rows;
  if (!make_row_tile_map(&fresh.map, base, rows, box_rows)) return false;
  slots[next++ % 32] = fresh;
  *out = fresh.map;
  return true;
}
}  // namespace

extern "C" size_t t2t_tile_attn_plan_ints(int H, int N, int CQ) {
  return plan_task_offset(H) + 4 * plan_max_tasks(H, N, CQ) + (size_t)H * CQ;
}

extern "C" size_t t2t_tile_attn_ws_bytes(int H, int N) {
  return (((size_t)H * N * kD * 2 + 255) & ~(size_t)255) + (size_t)H * N * 4;
}

static void split_ws(void* ws, int H, int N, __nv_bfloat16** attn_out, float** attn_lse) {
  *attn_out = (__nv_bfloat16*)ws;
  *attn_lse = (float*)((char*)ws + (((size_t)H * N * kD * 2 + 255) & ~(size_t)255));
}

extern "C" int t2t_tile_attn_plan(const void* tile_sizes, const void* kcounts, const void* unip, int* plan, int H,
                                  int N, int CQ, cudaStream_t st) {
  if (!tile_sizes || !kcounts || !unip || !plan || H <= 0 || N <= 0 || CQ <= 0) return T2T_ERR_ARG;
  const PlanView pv = plan_view(plan, H, N, CQ);
  if (cudaMemsetAsync(pv.counters, 0, PLAN_HDR * sizeof(int), st) != cudaSuccess) return T2T_ERR_CUDA;
  plan_kernel<<<H, 256, 0, st>>>((const int*)tile_sizes, (const int*)kcounts, (const uint32_t*)unip, H, N, CQ, plan);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}

extern "C" int t2t_tile_attn_exact(const void* q, const void* kp, const void* vp, const void* unip,
                                   const void* qperm, int* plan, int H, int N, int CQ, void* ws, size_t ws_bytes,
                                   int* d_status, cudaStream_t st) {
  return t2t_tile_attn_exact_strided(q, (long long)kD, (long long)N * kD, kp, vp, unip, qperm, plan, H, N, CQ, ws,
                                     ws_bytes, d_status, st);
}

extern "C" int t2t_tile_attn_exact_strided(const void* q, long long q_row_stride, long long q_head_stride,
                                           const void* kp, const void* vp, const void* unip, const void* qperm,
                                           int* plan, int H, int N, int CQ, void* ws, size_t ws_bytes,
                                           int* d_status, cudaStream_t st) {
  if (!q || !kp || !vp || !unip || !qperm || !plan || !ws || H <= 0 || N <= 0 || CQ <= 0) return T2T_ERR_ARG;
  // q rows are fetched by TMA row gathers from a [rows, 128] view of the tensor: whole rows between rows
  if (q_row_stride < kD || q_head_stride <= 0 || (q_row_stride % kD) || (q_head_stride % kD)) return T2T_ERR_ARG;
  const int q_row_step = (int)(q_row_stride / kD), q_head_step = (int)(q_head_stride / kD);
  const uint64_t q_rows = (uint64_t)(H - 1) * q_head_step + (uint64_t)(N - 1) * q_row_step + 1;
  if (ws_bytes < t2t_tile_attn_ws_bytes(H, N)) return T2T_ERR_WORKSPACE;
  __nv_bfloat16* attn_out;
  float* attn_lse;
  split_ws(ws, H, N, &attn_out, &attn_lse);
  const PlanView pv = plan_view(plan, H, N, CQ);
  // the task cursor is the only per-dispatch state of a prepared plan
  if (cudaMemsetAsync(pv.counters + 1, 0, sizeof(int), st) != cudaSuccess ||
      cudaMemsetAsync(pv.counters + 4, 0, sizeof(int), st) != cudaSuccess)
    return T2T_ERR_CUDA;
  const DeviceFacts* facts = device_facts();
  if (!facts) return T2T_ERR_CUDA;
  const int sms = facts->sms;
  // tensor maps over q, kp, vp as [H * N, 128] matrices: the kernel fetches tile rows four at a time
  CUtensorMap mq;
  KVMaps kv;
  const uint64_t rows = (uint64_t)H * (uint64_t)N;
  if (!cached_row_map(&mq, q, q_rows, 1) || !cached_row_map(&kv.k1, kp, rows, 1) ||
      !cached_row_map(&kv.k32, kp, rows, 32) || !cached_row_map(&kv.k64, kp, rows, 64) ||
      !cached_row_map(&kv.v1, vp, rows, 1) || !cached_row_map(&kv.v32, vp, rows, 32) ||
      !cached_row_map(&kv.v64, vp, rows, 64))
    return T2T_ERR_CUDA;
  // tasks above 128 rows first (one CTA per SM, two row tiles per K/V stream), then the others
  attn2_kernel<<<sms, A2_THREADS, A2_SMEM, st>>>(mq, kv, (const uint32_t*)unip, (const int*)qperm, attn_out,
                                                 attn_lse, plan, H, N, CQ, q_row_step, q_head_step, d_status);
  // The two kernels take disjoint tasks (own cursors, own output rows), so the second may start while the
  // first drains: it is launched with programmatic stream serialization and the first kernel releases its
  // dependents at once.  Their CTAs cannot share an SM (shared memory), so the second kernel's CTAs move in
  // as the first kernel's CTAs run out of tasks and exit.  Later work in the stream waits for both as usual.
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * sms);
  cfg.blockDim = dim3(A1_THREADS);
  cfg.dynamicSmemBytes = A1_SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, attn_kernel, mq, kv, (const uint32_t*)unip, (const int*)qperm, attn_out, attn_lse,
                         plan, H, N, CQ, q_row_step, q_head_step, d_status) != cudaSuccess)
    return T2T_ERR_CUDA;
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}

extern "C" int t2t_tile_attn_merge(const void* QU, const void* cks, const void* sumv, const void* kcounts,
                                   const void* unip, const void* qlab, const void* qperm, const void* lam,
                                   const float* tailw, void* out, int H, int N, int CQ, void* ws, size_t ws_bytes,
                                   int* d_status, cudaStream_t st) {
  return t2t_tile_attn_merge_strided(QU, cks, sumv, kcounts, unip, qlab, qperm, lam, tailw, out, (long long)kD,
                                     (long long)N * kD, H, N, CQ, ws, ws_bytes, d_status, st);
}

extern "C" int t2t_tile_attn_merge_strided(const void* QU, const void* cks, const void* sumv, const void* kcounts,
                                           const void* unip, const void* qlab, const void* qperm, const void* lam,
                                           const float* tailw, void* out, long long out_row_stride,
                                           long long out_head_stride, int H, int N, int CQ, void* ws,
                                           size_t ws_bytes, int* d_status, cudaStream_t st) {
  if (!QU || !cks || !sumv || !kcounts || !unip || !qlab || !qperm || !lam || !tailw || !out || !ws)
    return T2T_ERR_ARG;
  if (H <= 0 || N <= 0 || CQ <= 0) return T2T_ERR_ARG;
  if (out_row_stride < kD || out_head_stride <= 0 || (out_row_stride & 7) || (out_head_stride & 7)) return T2T_ERR_ARG;
  if (ws_bytes < t2t_tile_attn_ws_bytes(H, N)) return T2T_ERR_WORKSPACE;
  __nv_bfloat16* attn_out;
  float* attn_lse;
  split_ws(ws, H, N, &attn_out, &attn_lse);
  if (!device_facts()) return T2T_ERR_CUDA;
  // the value sums as an [H * 2048, 128] matrix, fetched 64 rows x 64 columns at a time
  CUtensorMap msv;
  if (!cached_row_map(&msv, sumv, (uint64_t)H * kC, TL_H)) return T2T_ERR_CUDA;
  tail_kernel<<<dim3(cdiv(N, TL_Q), H), TL_THREADS, TL_SMEM, st>>>(
      msv, attn_out, attn_lse, (const __nv_bfloat16*)QU, (const __nv_bfloat16*)cks, (const int*)kcounts, (const uint32_t*)unip, (const int*)qlab, (const int*)qperm, (const float*)lam, tailw,
      (__nv_bfloat16*)out, out_row_stride, out_head_stride, N, CQ, d_status);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}

extern "C" int t2t_tile_attn(const void* q, const void* kp, const void* vp, const void* tile_sizes,
                             const void* kcounts, const void* unip, const void* QU, const void* cks,
                             const void* sumv, const void* lam, const void* qlab, const void* qperm,
                             const float* tailw, void* out, int* plan, int rebuild_plan, int H, int N, int CQ,
                             void* ws, size_t ws_bytes, int* d_status, cudaStream_t st) {
  int rc = T2T_OK;
  if (rebuild_plan) rc = t2t_tile_attn_plan(tile_sizes, kcounts, unip, plan, H, N, CQ, st);
  if (rc == T2T_OK) rc = t2t_tile_attn_exact(q, kp, vp, unip, qperm, plan, H, N, CQ, ws, ws_bytes, d_status, st);
  if (rc == T2T_OK)
    rc = t2t_tile_attn_merge(QU, cks, sumv, kcounts, unip, qlab, qperm, lam, tailw, out, H, N, CQ, ws, ws_bytes,
                             d_status, st);
  return rc;
}

extern "C" int t2t_tile_attn_plan_info(const int* plan, int H, int N, int CQ, int* d_info, cudaStream_t st) {
  if (!plan || !d_info) return T2T_ERR_ARG;
  const PlanView pv = plan_view(const_cast<int*>(plan), H, N, CQ);
  plan_info_kernel<<<1, 32, 0, st>>>(pv.counters, d_info);
  return cudaGetLastError() == cudaSuccess ? T2T_OK : T2T_ERR_CUDA;
}
