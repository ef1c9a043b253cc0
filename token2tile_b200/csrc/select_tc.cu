// Scoring + budgeted cluster selection + union on the tensor cores.
//
// The selection of a query is DEFINED on exact scores (fp32 fused-multiply-add
// chain over k, rounded to fp16; see select.cu).  Evaluating 2048 chains per
// query costs N * C * 32 FMAs.  Here one CTA owns 128 consecutive rows of the
// cluster-sorted query order (a tile may span several query clusters: the rows
// of cluster k form "segment" k of the tile and selections are OR-ed into the
// segment's bitmap, flushed to the cluster's bitmap at the end).  A tcgen05 MMA
// (128 x 128 x 32 per chunk of centroids, all 2048 centroids resident in shared
// memory) gives approximate scores s~ in TMEM, and each row is settled in three
// steps, two of them streaming passes over the scores:
//
//   P1  row mean and deviation from the head's centroid moments (q . mean centroid,
//       q^T (mean c c^T) q): no pass; the scores lie in [-||q|| max ||c||, ||q|| max ||c||];
//   P2  size-weighted histogram of s~ over [mean, max] (refined if the threshold
//       bucket is crowded) -> the bucket [x_lo, x_hi] in which the running token
//       count first reaches ns;
//   P3  clusters with s~ > x_hi + 2 e' are selected outright (their sizes are
//       summed exactly), clusters with s~ in [x_lo - 2 e', x_hi + 2 e'] become
//       candidates; candidates get their exact chain score and fp16 key and are
//       walked in (key descending, index ascending) order until ns is reached.
//
// With |s~ - chain| <= e_i (see assign_tc.cu for the bound; e_i = 2^-14 ||q_i||
// max_c ||cks_c||) and e' = e_i + half an fp16 ulp at the threshold, every
// cluster above the window is strictly above the exact threshold key and every
// cluster below it strictly below, so the result equals the all-exact rule bit
// for bit.  Rows that do not fit the fast path (more than 64 candidates, no
// convergence, non-finite scores) are queued for the exact warp-per-row kernel.
#include "common.cuh"
#include "internal.h"

namespace t2t {

constexpr int ST_THREADS = 512;
constexpr int ST_CH = 64;                  // centroids per MMA chunk
constexpr int ST_NCH = kC / ST_CH;         // 32: eight per column group, double-buffered in TMEM
constexpr int ST_B = 64;                   // histogram buckets
constexpr int ST_CAP = 64;                 // candidates per row
constexpr int ST_REFINE = 40;              // refine the bucket when it alone holds more clusters than this
constexpr int ST_MAX_ITERS = 5;
constexpr int kMomFloats = 32 + 32 * 32;   // per head: mean centroid, second-moment matrix
constexpr int kMomParts = 8;               // the moments are summed over this many slices of the centroids
constexpr int ST_TPC = 4;                  // consecutive 128-row tiles of one head per CTA: the head's centroids, sizes
                                           // and prefix sums are staged once for all of them
constexpr int ST_STRAGGLERS = 8;           // this few unsettled rows of a tile go to the exact kernel instead of another pass

constexpr int OFF_CK = 0;                               // 1024 rows x 128 B: centroid c in row c % 1024, half c / 1024
constexpr int OFF_A = OFF_CK + 1024 * 128;              // 128 rows x 128 B (first 64 B used)
constexpr int OFF_HIST = OFF_A + 128 * 128;             // [ST_B][128] packed (size << 12 | count); after P2 the
constexpr int OFF_CAND = OFF_HIST;                      //   same bytes hold [128][ST_CAP] cluster | key << 16
constexpr int OFF_SIZE = OFF_HIST + ST_B * 128 * 4;     // [2048] (cluster size << 12) + 1
constexpr int OFF_PART = OFF_SIZE + kC * 4;             // [3][4][128] per-group partial max / sum / sum of squares
constexpr int OFF_ROW = OFF_PART + 12 * 128 * 4;        // [17][128] per-row scalars
constexpr int ST_MAXSEG = 8;                            // query clusters one tile may span on the fast path
constexpr int ST_MAXCQ = 2048;                          // prefix sums of the query-cluster sizes live in smem
constexpr int OFF_UNION = OFF_ROW + 17 * 128 * 4;       // [ST_MAXSEG][64] segment bitmaps
constexpr int OFF_PRE = OFF_UNION + ST_MAXSEG * 64 * 4; // [ST_MAXCQ + 1] first sorted row of every query cluster
constexpr int OFF_MISC = OFF_PRE + (ST_MAXCQ + 4) * 4;  // barriers, segment tables, ...
constexpr int OFF_MOM = OFF_MISC + 512;                 // [kMomFloats] the head's centroid moments
constexpr int ST_SMEM = OFF_MOM + kMomFloats * 4 + 1024;
static_assert(ST_SMEM <= 227 * 1024, "shared memory of select_tc_kernel");

// RS_QUEUE + k: queued for the exact kernel; k says why (1 non-finite scores, 2 threshold not bracketed,
// 3 too many candidates, 4 budget met above the window, 5 / 6 threshold outside the window, 7 walk ran dry,
// 8 the tile spans more query clusters than it has segment bitmaps)
enum : int { RS_SEARCH = 0, RS_COLLECT = 1, RS_DONE = 2, RS_QUEUE = 3, RS_WALK = 16 };
// per-row scalar slots
enum : int { R_LO = 0, R_HI, R_INV, R_THRA, R_THRW, R_EPS, R_MIN, R_CUM, R_STATE, R_NCAND, R_SIZEA, R_ORIG, R_E2, R_CLU, R_SEG, R_OVF, R_MAX };

__device__ __forceinline__ int key16_from_half(__half hv) {
  unsigned u = __half_as_ushort(hv);
  u ^= ((u >> 15) & 1u) * 0x7FFFu;
  return (int)((u ^ 0x8000u) & 0xFFFFu);
}
__device__ __forceinline__ int key16_from_score(float s) { return key16_from_half(__float2half_rn(s)); }

// Candidate slot `slot` of row r: the slot index is rotated by the row so that the rows of a warp, reading the
// same slot, hit 32 different banks (the row stride, ST_CAP words, is a multiple of the bank count).
__device__ __forceinline__ int cand_at(int r, int slot) { return r * ST_CAP + ((slot + r) & (ST_CAP - 1)); }

__device__ __forceinline__ void wg_sync(int g) { asm volatile("bar.sync %0, 128;" ::"r"(g + 1) : "memory"); }

__global__ void __launch_bounds__(ST_THREADS, 1) select_tc_kernel(
    const __nv_bfloat16* __restrict__ QU, const __nv_bfloat16* __restrict__ cks,
    const int* __restrict__ kcounts, const int* __restrict__ qperm, const int* __restrict__ tile_sizes,
    const int* __restrict__ ns_ptr, int* __restrict__ unip, int* __restrict__ rowcnt, int N, int CQ,
    int* __restrict__ fixq, const float* __restrict__ mom, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sm = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t sCk = base + OFF_CK, sA = base + OFF_A;
  int* sHist = reinterpret_cast<int*>(sm + OFF_HIST);
  uint32_t* sCand = reinterpret_cast<uint32_t*>(sm + OFF_CAND);
  int* sSizeP = reinterpret_cast<int*>(sm + OFF_SIZE);
  float* sPart = reinterpret_cast<float*>(sm + OFF_PART);
  float* sRowF = reinterpret_cast<float*>(sm + OFF_ROW);
  int* sRowI = reinterpret_cast<int*>(sm + OFF_ROW);
  uint32_t* sUnion = reinterpret_cast<uint32_t*>(sm + OFF_UNION);             // [ST_MAXSEG][64]
  int* sPre = reinterpret_cast<int*>(sm + OFF_PRE);                           // [CQ + 1]
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + OFF_MISC);                // [4 groups][2 buffers]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sm + OFF_MISC + 320);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(sm + OFF_MISC + 324);
  int* sCmax = reinterpret_cast<int*>(sm + OFF_MISC + 328);                    // max ||cks||^2 as int bits
  int* sScan = reinterpret_cast<int*>(sm + OFF_MISC + 64);                    // [16] scan scratch
  int* sSegClu = reinterpret_cast<int*>(sm + OFF_MISC + 128);                 // [ST_MAXSEG] cluster of each segment
  uint32_t* sSegMask = reinterpret_cast<uint32_t*>(sm + OFF_MISC + 160);      // [4 warps][ST_MAXSEG] lanes of a segment
  int* sNseg = reinterpret_cast<int*>(sm + OFF_MISC + 288);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = tid >> 7;            // column group: chunks g, g + 4, g + 8, ...
  const int r = tid & 127;           // row of the tile = TMEM lane
  const int h = blockIdx.y;
  const __nv_bfloat16* ckh = cks + (size_t)h * kC * kR;

  if (warp == 0) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  if (tid == 0) {
    *abort_flag = 0;
    *sCmax = 0;
    for (int i = 0; i < 8; ++i) mbar_init(bars + i, 1);
    mbar_init_fence();
  }
  sUnion[tid] = 0u;                                     // ST_MAXSEG * 64 == ST_THREADS words
  // all 2048 centroids: 16-byte chunk id -> centroid id >> 2, chunk id & 3
#pragma unroll
  for (int i = 0; i < (kC * 4) / ST_THREADS; ++i) {
    const int id = tid + ST_THREADS * i;
    const int c = id >> 2, ch = id & 3;
    cp_async16(sCk + sw128(c & 1023, (c >> 10) * 4 + ch), ckh + (size_t)c * kR + ch * 8, 16u);
  }
  cp_async_commit();
  for (int c = tid; c < kC; c += ST_THREADS) sSizeP[c] = (kcounts[(size_t)h * kC + c] << 12) + 1;
  float* sMom = reinterpret_cast<float*>(sm + OFF_MOM);
  for (int i = tid; i < kMomFloats; i += ST_THREADS) {      // slices added in a fixed order
    float acc = 0.f;
#pragma unroll
    for (int p = 0; p < kMomParts; ++p) acc += mom[((size_t)h * kMomParts + p) * kMomFloats + i];
    sMom[i] = acc;
  }
  __syncthreads();
  {
    // exclusive prefix sums of the query-cluster sizes
    int carry = 0;
    for (int c0 = 0; c0 < CQ; c0 += ST_THREADS) {
      const int c = c0 + tid;
      const int v = c < CQ ? tile_sizes[(size_t)h * CQ + c] : 0;
      const int inc = warp_incl_scan(v, lane);
      if (lane == 31) sScan[warp] = inc;
      __syncthreads();
      int wbase = 0;
      for (int w = 0; w < warp; ++w) wbase += sScan[w];
      if (c < CQ) sPre[c] = carry + wbase + inc - v;
      int tot = 0;
      for (int w = 0; w < ST_THREADS / 32; ++w) tot += sScan[w];
      carry += tot;
      __syncthreads();
    }
    if (tid == 0) sPre[CQ] = carry;
  }
  cp_async_wait<0>();
  __syncthreads();
  {
    // largest squared norm of a scoring centroid
    float mx = 0.f;
    for (int c = tid; c < kC; c += ST_THREADS) {
      float s = 0.f;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint4 w = *reinterpret_cast<const uint4*>(sm + OFF_CK + sw128(c & 1023, (c >> 10) * 4 + q4));
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          s = fmaf(bf_lo(ws[e]), bf_lo(ws[e]), s);
          s = fmaf(bf_hi(ws[e]), bf_hi(ws[e]), s);
        }
      }
      mx = fmaxf(mx, s);
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
    if (lane == 0) atomicMax(sCmax, __float_as_int(mx));
  }
  fence_proxy_async();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t t_lane = tmem_addr(tmem, (warp & 3) * 32, g * 2 * ST_CH);      // two buffers of ST_CH columns
  const int ns = *ns_ptr;
  const float cmaxnorm = sqrtf(__int_as_float(*sCmax));
  constexpr uint32_t idesc = make_idesc_bf16(128, ST_CH, false, false);
  uint32_t ph0 = 0, ph1 = 0;        // phases of this group's two buffer barriers
  bool dead = false;

  // Streams this group's eight chunks through its two TMEM buffers: the MMA of
  // chunk i + 1 runs while chunk i is scanned.  body(cbase, v) sees 32
  // consecutive approximate scores of this thread's row.
  auto issue = [&](int i) {        // called by the group's first thread
    const int cc = g + 4 * i, b = i & 1;
    tc_fence_after();
#pragma unroll
    for (int s2 = 0; s2 < 2; ++s2)
      umma_ss(tmem + g * 2 * ST_CH + b * ST_CH, make_sdesc(sA + s2 * 32, 16, 1024),
              make_sdesc(sCk + (cc & 15) * (ST_CH * 128) + (cc >> 4) * 64 + s2 * 32, 16, 1024), idesc,
              s2 > 0 ? 1u : 0u);
    umma_commit(bars + g * 2 + b);
  };
  auto stream = [&](auto&& body) {
    if (dead) return;
    if (r == 0) issue(0);
#pragma unroll 1
    for (int i = 0; i < ST_NCH / 4; ++i) {
      const int cc = g + 4 * i, b = i & 1;
      // every warp of the group has finished reading the other buffer (chunk i - 1): refill it
      tc_fence_before();
      wg_sync(g);
      if (r == 0 && i + 1 < ST_NCH / 4) issue(i + 1);
      if (!mbar_wait(bars + g * 2 + b, b ? ph1 : ph0, abort_flag)) { dead = true; break; }
      if (b) ph1 ^= 1u; else ph0 ^= 1u;
      tc_fence_after();
#pragma unroll 1      // keeps each pass body at 32 columns of code; fully unrolled the kernel outgrows the I-cache
      for (int q = 0; q < ST_CH / 32; ++q) {
        uint32_t v[32];
        tmem_ld32(t_lane + b * ST_CH + q * 32, v);
        tmem_wait_ld();
        body(cc * ST_CH + q * 32, v);
      }
    }
    tc_fence_before();
    wg_sync(g);
  };

#pragma unroll 1
  for (int ti = 0; ti < ST_TPC; ++ti) {
    const int p0 = (blockIdx.x * ST_TPC + ti) * 128;    // first sorted row of this tile
    if (p0 >= N || dead) break;
    const int rows_here = min(128, N - p0);
    {
      const int ar = tid >> 2, ch = tid & 3;
      const bool valid = ar < rows_here;
      const int orig = valid ? qperm[(size_t)h * N + p0 + ar] : 0;
      cp_async16(sA + sw128(ar, ch), QU + ((size_t)h * N + orig) * kR + ch * 8, valid ? 16u : 0u);
      cp_async_commit();
      if (ch == 0) sRowI[R_ORIG * 128 + ar] = orig;
    }
    if (g == 0) {
      // query cluster of this sorted row: the last t with sPre[t] <= p (empty clusters are skipped)
      int lo = 0, hi = CQ;                               // invariant: sPre[lo] <= p < sPre[hi]
      const int p = p0 + (r < rows_here ? r : rows_here - 1);
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (sPre[mid] <= p) lo = mid; else hi = mid;
      }
      sRowI[R_CLU * 128 + r] = lo;
    }
    cp_async_wait<0>();
    fence_proxy_async();
    tc_fence_before();
    __syncthreads();
    if (g == 0) {
      // segment of the row = number of cluster changes before it
      const int clu = sRowI[R_CLU * 128 + r];
      const int flag = (r > 0 && sRowI[R_CLU * 128 + r - 1] != clu) ? 1 : 0;
      const int inc = warp_incl_scan(flag, lane);
      if (lane == 31) sScan[warp] = inc;
      wg_sync(0);
      int seg = inc;
      for (int w = 0; w < warp; ++w) seg += sScan[w];
      sRowI[R_SEG * 128 + r] = seg;
      if (seg < ST_MAXSEG && (flag || r == 0)) sSegClu[seg] = clu;
      if (r == 127) *sNseg = seg + 1 < ST_MAXSEG ? seg + 1 : ST_MAXSEG;
#pragma unroll
      for (int k = 0; k < ST_MAXSEG; ++k) {
        const uint32_t m = __ballot_sync(0xffffffffu, seg == k && r < rows_here);
        if (lane == 0) sSegMask[warp * ST_MAXSEG + k] = m;
      }
    }
    if (g == 0) {
      float qn = 0.f;
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint4 w = *reinterpret_cast<const uint4*>(sm + OFF_A + sw128(r, q4));
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          qn = fmaf(bf_lo(ws[e]), bf_lo(ws[e]), qn);
          qn = fmaf(bf_hi(ws[e]), bf_hi(ws[e]), qn);
        }
      }
      const float bound = sqrtf(qn) * cmaxnorm;
      sRowF[R_MAX * 128 + r] = bound;            // no score exceeds ||q|| max ||c||
      sRowF[R_EPS * 128 + r] = 6.103515625e-05f * bound + 1.0e-30f;
      sRowF[R_MIN * 128 + r] = -bound - 1.0f;
      sRowI[R_STATE * 128 + r] =
          r < rows_here ? (sRowI[R_SEG * 128 + r] < ST_MAXSEG ? RS_SEARCH : RS_QUEUE + 8) : RS_DONE;
      sRowI[R_CUM * 128 + r] = 0;
      sRowI[R_NCAND * 128 + r] = 0;
      sRowI[R_SIZEA * 128 + r] = 0;
    }

    // ---- P1: mean and standard deviation of the row's scores, without a pass over them ------------
    // sum_c q.c = q . sum_c c and sum_c (q.c)^2 = q^T (sum_c c c^T) q: the head's centroid moments (a
    // 32-vector and a 32 x 32 matrix, fp32) give both in 1056 multiply-adds per row.  Each column group
    // takes eight rows of the matrix.  The statistics only place the first histogram range.
    {
      const float* mh = sMom;
      float qv[32];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint4 w = *reinterpret_cast<const uint4*>(sm + OFF_A + sw128(r, q4));
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { qv[q4 * 8 + 2 * e] = bf_lo(ws[e]); qv[q4 * 8 + 2 * e + 1] = bf_hi(ws[e]); }
      }
      float qa[8];      // elements 8 g .. 8 g + 7 of the row: chunk g
      {
        const uint4 w = *reinterpret_cast<const uint4*>(sm + OFF_A + sw128(r, g));
        const uint32_t ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) { qa[2 * e] = bf_lo(ws[e]); qa[2 * e + 1] = bf_hi(ws[e]); }
      }
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4* grow = reinterpret_cast<const float4*>(mh + 32 + (8 * g + i) * 32);
        float t0 = 0.f, t1 = 0.f;
#pragma unroll
        for (int b4 = 0; b4 < 8; ++b4) {
          const float4 mm = grow[b4];      // the same address in every thread of the group: a broadcast
          t0 = fmaf(mm.x, qv[4 * b4], t0);
          t1 = fmaf(mm.y, qv[4 * b4 + 1], t1);
          t0 = fmaf(mm.z, qv[4 * b4 + 2], t0);
          t1 = fmaf(mm.w, qv[4 * b4 + 3], t1);
        }
        s2 = fmaf(qa[i], t0 + t1, s2);
        s1 = fmaf(qa[i], mh[8 * g + i], s1);
      }
      sPart[(1 * 4 + g) * 128 + r] = s1;
      sPart[(2 * 4 + g) * 128 + r] = s2;
    }
    __syncthreads();
    if (g == 0 && sRowI[R_STATE * 128 + r] == RS_SEARCH) {
      float mean = 0.f, s2 = 0.f;
#pragma unroll
      for (int gg = 0; gg < 4; ++gg) {
        mean += sPart[(1 * 4 + gg) * 128 + r];
        s2 += sPart[(2 * 4 + gg) * 128 + r];
      }
      const float M = sRowF[R_MAX * 128 + r];
      const float sd = sqrtf(fmaxf(s2 - mean * mean, 1.0e-20f));
      const bool finite = fabsf(M) < INFINITY && fabsf(s2) < INFINITY && fabsf(mean) < INFINITY;
      // First range: 2.5 standard deviations around the score a fraction ns / N of a bell-shaped
      // distribution would exceed (inverse normal tail, Abramowitz-Stegun 26.2.23).  Everything above the
      // range is counted in an overflow bucket.  The range only has to be a good guess: the search continues
      // above it (up to the bound ||q|| max ||c||) or below it when the running token count says so.
      const float f = fminf(0.5f, fmaxf((float)ns / (float)N, 1.0e-6f));
      const float tt = sqrtf(-2.0f * __logf(f));
      const float z = tt - (2.515517f + tt * (0.802853f + tt * 0.010328f)) /
                               (1.0f + tt * (1.432788f + tt * (0.189269f + tt * 0.001308f)));
      float hi = mean + (z + 1.25f) * sd;
      const int ovf = hi < M ? 1 : 0;
      hi = ovf ? hi : M;
      const float lo = fminf(mean + (z - 1.25f) * sd, hi);
      sRowF[R_HI * 128 + r] = hi;
      sRowF[R_LO * 128 + r] = lo;
      sRowI[R_OVF * 128 + r] = ovf;
      sRowF[R_INV * 128 + r] = hi > lo ? (float)(ST_B - ovf) / (hi - lo) : 0.f;
      if (!finite) sRowI[R_STATE * 128 + r] = RS_QUEUE + 1;
    }

    // ---- P2: histogram search for the threshold bucket --------------------------
    for (int it = 0; it < ST_MAX_ITERS; ++it) {
      for (int i = tid; i < ST_B * 128; i += ST_THREADS) sHist[i] = 0;
      __syncthreads();
      {
        // bucket = floor((hi - s) * inv): s > hi gives a negative bucket; rows that are not searching get
        // hi = -inf and fall out the same way
        const bool act = sRowI[R_STATE * 128 + r] == RS_SEARCH;
        const float hi = act ? sRowF[R_HI * 128 + r] : -INFINITY;
        const float inv = act ? sRowF[R_INV * 128 + r] : 1.0f;
        const float ninv = -inv, hiinv = hi * inv;
        // with an overflow bucket, bucket 0 takes every score above hi and the range starts at bucket 1
        const int ovf = act ? sRowI[R_OVF * 128 + r] : 0;
        const int bmin = ovf - 1;
        int* hist_r = sHist + r;
        stream([&](int cbase, const uint32_t(&v)[32]) {
#pragma unroll
          for (int j4 = 0; j4 < 32; j4 += 4) {
            const int4 p4 = *reinterpret_cast<const int4*>(sSizeP + cbase + j4);
            const int pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              // floor by an add rounded toward -inf: 1.5 * 2^23 + t has floor(t) in its low mantissa bits for
              // |t| < 2^22; beyond that the difference keeps the sign of t and is far outside [0, ST_B).
              // t = (hi - s) inv as one multiply-add: a score within a rounding step of a bucket boundary may
              // land in the neighbouring bucket, which only moves the window (the selection is validated
              // against exact keys afterwards)
              const float t = __fmaf_rd(__uint_as_float(v[j4 + e]), ninv, hiinv);
              const int b = max(__float_as_int(__fadd_rd(t, 12582912.0f)) - 0x4B400000 + ovf, bmin);
              if ((unsigned)b < (unsigned)ST_B) atomicAdd(hist_r + b * 128, pp[e]);
            }
          }
        });
      }
      __syncthreads();
      int searching = 0;
      if (g == 0 && sRowI[R_STATE * 128 + r] == RS_SEARCH) {
        const float hi = sRowF[R_HI * 128 + r], lo = sRowF[R_LO * 128 + r];
        const float eps = sRowF[R_EPS * 128 + r];
        const int ovf = sRowI[R_OVF * 128 + r];
        int cum = sRowI[R_CUM * 128 + r];
        int bstar = -1, cnt = 0;
        bool above = false;                       // the budget is met inside the overflow bucket
        if (ovf) {
          const int p = sHist[r];
          if (cum + (p >> 12) >= ns) above = true; else cum += p >> 12;
        }
        for (int b = ovf; b < ST_B && !above; ++b) {
          const int p = sHist[b * 128 + r];
          if (cum + (p >> 12) >= ns) { bstar = b - ovf; cnt = p & 4095; break; }
          cum += p >> 12;
        }
        const float w = (hi - lo) / (float)(ST_B - ovf);
        if (above) {
          // continue between hi and the row maximum (nothing has been added to cum)
          if (it + 1 < ST_MAX_ITERS) {
            const float M = sRowF[R_MAX * 128 + r];
            sRowF[R_LO * 128 + r] = hi;
            sRowF[R_HI * 128 + r] = M;
            sRowI[R_OVF * 128 + r] = 0;
            sRowF[R_INV * 128 + r] = M > hi ? (float)ST_B / (M - hi) : 0.f;
            searching = 1;
          } else {
            sRowI[R_STATE * 128 + r] = RS_QUEUE + 2;
          }
        } else
        if (bstar < 0) {
          // the threshold lies below this range: continue from its lower end down to the next floor
          // (first the row mean, then the lower bound -||q|| max ||c|| of any score)
          const float mn = sRowF[R_MIN * 128 + r];
          if (lo > mn && it + 1 < ST_MAX_ITERS) {
            sRowI[R_CUM * 128 + r] = cum;
            sRowF[R_HI * 128 + r] = lo;
            sRowF[R_LO * 128 + r] = mn;
            sRowF[R_INV * 128 + r] = (float)ST_B / (lo - mn);
            sRowI[R_OVF * 128 + r] = 0;
            sRowF[R_MIN * 128 + r] = lo;               // no further floor: a second miss goes to the exact kernel
            searching = 1;
          } else {
            sRowI[R_STATE * 128 + r] = RS_QUEUE + 2;
          }
        } else {
          const float x_hi = hi - (float)bstar * w, x_lo = hi - (float)(bstar + 1) * w;
          // 2^-10 |x|: half an fp16 ulp even if the threshold sits just across a power of two
          const float e2 = 2.0f * (eps + 9.765625e-04f * fmaxf(fabsf(x_lo), fabsf(x_hi)) + 5.9604645e-08f);
          if (cnt > ST_REFINE && it + 1 < ST_MAX_ITERS && w > 2.0f * e2) {
            sRowI[R_CUM * 128 + r] = cum;            // sizes above the bucket are settled
            sRowF[R_HI * 128 + r] = x_hi;
            sRowF[R_LO * 128 + r] = x_lo;
            sRowF[R_INV * 128 + r] = (float)ST_B / (x_hi - x_lo);
            sRowI[R_OVF * 128 + r] = 0;
            searching = 1;
          } else {
            sRowF[R_THRA * 128 + r] = x_hi + e2;
            sRowF[R_THRW * 128 + r] = x_lo - e2;
            sRowF[R_E2 * 128 + r] = e2;
            sRowI[R_STATE * 128 + r] = RS_COLLECT;
          }
        }
      }
      const int unsettled = __syncthreads_count(searching);
      if (unsettled == 0) break;
      if (unsettled <= ST_STRAGGLERS) {          // cheaper to hand a few rows to the exact kernel than to run a pass
        if (searching) sRowI[R_STATE * 128 + r] = RS_QUEUE + 2;
        break;
      }
    }
    if (g == 0 && sRowI[R_STATE * 128 + r] == RS_SEARCH) sRowI[R_STATE * 128 + r] = RS_QUEUE + 2;
    __syncthreads();

    // ---- P3: select above the window, collect candidates inside it ---------------
    {
      const bool act = sRowI[R_STATE * 128 + r] == RS_COLLECT;
      const float thrA = act ? sRowF[R_THRA * 128 + r] : INFINITY;
      const float thrW = act ? sRowF[R_THRW * 128 + r] : INFINITY;
      int sumA = 0;      // packed: (sizes << 12) + count
      const int nseg = *sNseg;
      const uint32_t* segmask = sSegMask + (warp & 3) * ST_MAXSEG;
      // segment of this warp's rows if they all share one (the common case), else -1
      int one_seg = -1;
      for (int k = 0; k < nseg; ++k)
        if (segmask[k] != 0u) one_seg = (one_seg == -1) ? k : -2;
      stream([&](int cbase, const uint32_t(&v)[32]) {
        // straight-line over the 32 scores: bit masks of the clusters above the window and of those at or
        // above its lower end; the (few) candidates are appended afterwards from the difference
        // The comparisons as sign bits of differences (a > thrA iff thrA - a < 0; a >= thrW iff not a - thrW < 0),
        // shifted into the masks from score 31 down to score 0: a subtraction on the FMA pipe and a funnel shift
        // per bit instead of a compare and a predicated OR on the half-rate ALU pipe.  (Rows that do not collect
        // have thrA = thrW = +inf: no bit of either mask.)
        uint32_t wbits = 0u, nbits = 0u;
#pragma unroll
        for (int j = 31; j >= 0; --j) {
          const float a = __uint_as_float(v[j]);
          wbits = __funnelshift_l(__float_as_uint(thrA - a), wbits, 1);
          nbits = __funnelshift_l(__float_as_uint(a - thrW), nbits, 1);
        }
        const uint32_t ibits = ~nbits;
        // sizes of the (few) clusters above the window
        for (uint32_t wb = wbits; wb; wb &= wb - 1u) sumA += sSizeP[cbase + __ffs(wb) - 1];
        uint32_t cbits = ibits & ~wbits;
        while (cbits) {
          const int j = __ffs(cbits) - 1;
          cbits &= cbits - 1u;
          const int slot = atomicAdd(&sRowI[R_NCAND * 128 + r], 1);
          if (slot < ST_CAP) sCand[cand_at(r, slot)] = (uint32_t)(cbase + j);
        }
        // clusters some row of this warp takes outright -> the bitmap of the rows' segment(s)
        const uint32_t any = __reduce_or_sync(0xffffffffu, wbits);
        if (any) {
          if (one_seg >= 0) {
            uint32_t* w = sUnion + one_seg * 64 + (cbase >> 5);
            if (lane == 0 && (*w & any) != any) atomicOr(w, any);
          } else {
#pragma unroll 1
            for (int k = 0; k < nseg; ++k) {
              const uint32_t mine = (segmask[k] >> lane) & 1u ? wbits : 0u;
              const uint32_t segbits = __reduce_or_sync(0xffffffffu, mine);
              uint32_t* w = sUnion + k * 64 + (cbase >> 5);
              if (lane == 0 && segbits && (*w & segbits) != segbits) atomicOr(w, segbits);
            }
          }
        }
      });
      if (sumA) atomicAdd(&sRowI[R_SIZEA * 128 + r], sumA >> 12);
    }
    __syncthreads();

    // ---- exact keys of the candidates (four threads share a row) ------------------
    {
      const int st = sRowI[R_STATE * 128 + r];
      const int n = sRowI[R_NCAND * 128 + r];
      if (st == RS_COLLECT && n <= ST_CAP && g < n) {
        float q[kR];
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint4 w = *reinterpret_cast<const uint4*>(sm + OFF_A + sw128(r, q4));
          q[8 * q4 + 0] = bf_lo(w.x); q[8 * q4 + 1] = bf_hi(w.x);
          q[8 * q4 + 2] = bf_lo(w.y); q[8 * q4 + 3] = bf_hi(w.y);
          q[8 * q4 + 4] = bf_lo(w.z); q[8 * q4 + 5] = bf_hi(w.z);
          q[8 * q4 + 6] = bf_lo(w.w); q[8 * q4 + 7] = bf_hi(w.w);
        }
        for (int slot = g; slot < n; slot += 4) {
          const int c = (int)(sCand[cand_at(r, slot)] & 0xFFFFu);
          float acc = 0.f;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            const uint4 w = *reinterpret_cast<const uint4*>(sm + OFF_CK + sw128(c & 1023, (c >> 10) * 4 + q4));
            acc = fmaf(q[8 * q4 + 0], bf_lo(w.x), acc); acc = fmaf(q[8 * q4 + 1], bf_hi(w.x), acc);
            acc = fmaf(q[8 * q4 + 2], bf_lo(w.y), acc); acc = fmaf(q[8 * q4 + 3], bf_hi(w.y), acc);
            acc = fmaf(q[8 * q4 + 4], bf_lo(w.z), acc); acc = fmaf(q[8 * q4 + 5], bf_hi(w.z), acc);
            acc = fmaf(q[8 * q4 + 6], bf_lo(w.w), acc); acc = fmaf(q[8 * q4 + 7], bf_hi(w.w), acc);
          }
          sCand[cand_at(r, slot)] = (uint32_t)c | ((uint32_t)key16_from_score(acc) << 16);
        }
      }
    }
    __syncthreads();

    // ---- settle the candidates in exact order; queue what could not be settled -------
    // Walking the candidates in (key descending, index ascending) order until the budget is met selects
    // candidate j iff the tokens above the window plus the sizes of the candidates before j stay below ns.
    // "Before" is a comparison of the entries with their low 16 bits flipped, so every candidate can be
    // decided on its own: first one thread per row validates the window, then four threads per row take a
    // quarter of the candidates each.
    if (g == 0) {
      int st = sRowI[R_STATE * 128 + r];
      const int n = sRowI[R_NCAND * 128 + r];
      if (st == RS_COLLECT) {
        const int running = sRowI[R_SIZEA * 128 + r];
        // Independent of how the window was found, the result is exact iff the exact threshold key lies
        // inside it: fewer than ns tokens have a key >= y = thrA - e' (every cluster above the window does,
        // plus the candidates counted here), and at least ns have a key >= z = thrW + e'.
        int why = n > ST_CAP ? 3 : (running >= ns ? 4 : 0);
        if (!why) {
          const float e1 = 0.5f * sRowF[R_E2 * 128 + r];
          const uint32_t ky = (uint32_t)key16_from_half(__float2half_ru(sRowF[R_THRA * 128 + r] - e1));
          const uint32_t kz = (uint32_t)key16_from_half(__float2half_ru(sRowF[R_THRW * 128 + r] + e1));
          int sy = running, sz2 = running, tot = running;
          for (int s2 = 0; s2 < n; ++s2) {
            const uint32_t e = sCand[cand_at(r, s2)];
            const int szc = sSizeP[e & 0xFFFFu] >> 12;
            sy += (e >> 16) >= ky ? szc : 0;
            sz2 += (e >> 16) >= kz ? szc : 0;
            tot += szc;
          }
          // 7: the window does not reach the budget, let the exact kernel decide
          why = sy >= ns ? 5 : (sz2 < ns ? 6 : (tot < ns ? 7 : 0));
        }
        st = why ? RS_QUEUE + why : RS_WALK;
        sRowI[R_STATE * 128 + r] = st;
      }
      if (st >= RS_QUEUE && st != RS_WALK) {
        int* qh = fixq + (size_t)h * (2 * (size_t)N + 1);
        const int slot = atomicAdd(qh, 1);
        qh[1 + 2 * slot] = sRowI[R_ORIG * 128 + r];
        qh[2 + 2 * slot] = sRowI[R_CLU * 128 + r] | ((st - RS_QUEUE) << 24);      // the reason rides in the top byte
      }
    }
    __syncthreads();
    if (sRowI[R_STATE * 128 + r] == RS_WALK) {
      const int n = sRowI[R_NCAND * 128 + r];
      const int running = sRowI[R_SIZEA * 128 + r];
      uint32_t* myUnion = sUnion + (sRowI[R_SEG * 128 + r] & (ST_MAXSEG - 1)) * 64;
      for (int j = g; j < n; j += 4) {
        const uint32_t ej = sCand[cand_at(r, j)];
        const uint32_t oj = ej ^ 0xFFFFu;
        int before = running;
        for (int i = 0; i < n; ++i) {
          const uint32_t ei = sCand[cand_at(r, i)];
          before += (ei ^ 0xFFFFu) > oj ? sSizeP[ei & 0xFFFFu] >> 12 : 0;
        }
        if (before < ns) {
          const uint32_t cj = ej & 0xFFFFu;
          const uint32_t bit = 1u << (cj & 31);
          if (!(myUnion[cj >> 5] & bit)) atomicOr(&myUnion[cj >> 5], bit);
          const int after = before + (sSizeP[cj] >> 12);
          // exactly one candidate crosses the budget: its running count is the row's token count
          if (after >= ns) rowcnt[(size_t)h * N + sRowI[R_ORIG * 128 + r]] = after;
        }
      }
    }
    __syncthreads();
    {
      // segment bitmaps -> the (zero-initialised) bitmaps of their query clusters
      const int k = tid >> 6, w = tid & 63;
      const uint32_t bits = sUnion[tid];
      if (k < *sNseg && bits)
        atomicOr(reinterpret_cast<unsigned*>(unip) + ((size_t)h * CQ + sSegClu[k]) * 64 + w, bits);
      sUnion[tid] = 0u;      // each thread clears the word it has just flushed, for the next tile
    }
    __syncthreads();
  }
  if (*abort_flag && tid == 0 && status) atomicCAS(status, ST_OK, ST_WAIT_TIMEOUT);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 512);
}

// pin_tail: every query cluster executes the reserved last key cluster
__global__ void pin_bit_kernel(int* __restrict__ unip, int rows) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < rows) atomicOr(reinterpret_cast<unsigned*>(unip) + (size_t)i * 64 + 63, 0x80000000u);
}

// First two moments of a head's scaled key centroids, as kMomParts partial sums (one CTA per slice of
// C / kMomParts centroids): mom[h][p] = { sum_c c / C (32), sum_c c c^T / C (32 x 32) } over the slice.
__global__ void __launch_bounds__(1024) centroid_moments_kernel(const __nv_bfloat16* __restrict__ cks,
                                                                float* __restrict__ mom) {
  constexpr int SLICE = kC / kMomParts;
  __shared__ float sc[SLICE][kR + 1];
  const int h = blockIdx.y, part = blockIdx.x, a = threadIdx.x >> 5, b = threadIdx.x & 31;
  const __nv_bfloat16* ch = cks + ((size_t)h * kC + (size_t)part * SLICE) * kR;
  for (int i = threadIdx.x; i < SLICE * kR; i += 1024) sc[i >> 5][i & 31] = bf_to_f(ch[i]);      // coalesced
  __syncthreads();
  float g0 = 0.f, g1 = 0.f, m0 = 0.f;
#pragma unroll 4
  for (int c = 0; c < SLICE; c += 2) {
    g0 = fmaf(sc[c][a], sc[c][b], g0);
    g1 = fmaf(sc[c + 1][a], sc[c + 1][b], g1);
    m0 += sc[c][b] + sc[c + 1][b];
  }
  float* mh = mom + ((size_t)h * kMomParts + part) * kMomFloats;
  mh[32 + a * 32 + b] = (g0 + g1) * (1.0f / kC);
  if (a == 0) mh[b] = m0 * (1.0f / kC);
}

static size_t select_queue_bytes(int H, int N) { return ((size_t)H * (2 * (size_t)N + 1) * sizeof(int) + 255) & ~(size_t)255; }
size_t select_ws_bytes(int H, int N) { return select_queue_bytes(H, N) + (size_t)H * kMomParts * kMomFloats * sizeof(float); }

}  // namespace t2t

using namespace t2t;

extern "C" size_t t2t_score_select_union_ws_bytes(int H, int N) { return select_ws_bytes(H, N); }

extern "C" int t2t_score_select_union(const void* QU, const void* cks, const void* kcounts, const void* qperm,
                                      const void* tile_sizes, const int* ns, void* unip, void* rowcnt, int H,
                                      int N, int CQ, int pin_tail, void* ws, size_t ws_bytes, int* d_status,
                                      cudaStream_t st) {
  if (!QU || !cks || !kcounts || !qperm || !tile_sizes || !ns || !unip || !rowcnt || !ws) return T2T_ERR_ARG;
  if (H <= 0 || N <= 0 || CQ <= 0 || N >= (1 << 19)) return T2T_ERR_ARG;
  if (ws_bytes < select_ws_bytes(H, N)) return T2T_ERR_WORKSPACE;
  if (CQ > ST_MAXCQ)      // the prefix sums of the query clusters would not fit: all-exact path
    return t2t_score_select_union_exact(QU, cks, kcounts, qperm, tile_sizes, ns, unip, rowcnt, H, N, CQ, pin_tail,
                                        st);
  int* fixq = (int*)ws;
  float* mom = reinterpret_cast<float*>((char*)ws + select_queue_bytes(H, N));
  centroid_moments_kernel<<<dim3(kMomParts, H), 1024, 0, st>>>((const __nv_bfloat16*)cks, mom);
  if (cudaMemsetAsync(fixq, 0, select_queue_bytes(H, N), st) != cudaSuccess ||
      cudaMemsetAsync(unip, 0, (size_t)H * CQ * 64 * sizeof(int), st) != cudaSuccess)
    return T2T_ERR_CUDA;
  if (cudaFuncSetAttribute(select_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM) != cudaSuccess)
    return T2T_ERR_CUDA;
  select_tc_kernel<<<dim3(cdiv(cdiv(N, 128), ST_TPC), H), ST_THREADS, ST_SMEM, st>>>(
      (const __nv_bfloat16*)QU, (const __nv_bfloat16*)cks, (const int*)kcounts, (const int*)qperm,
      (const int*)tile_sizes, ns, (int*)unip, (int*)rowcnt, N, CQ, fixq, mom, d_status);
  if (pin_tail > 0) pin_bit_kernel<<<cdiv(H * CQ, 256), 256, 0, st>>>((int*)unip, H * CQ);
  if (cudaGetLastError() != cudaSuccess) return T2T_ERR_CUDA;
  return launch_select_fix((const __nv_bfloat16*)QU, (const __nv_bfloat16*)cks, (const int*)kcounts, ns, (int*)unip,
                           (int*)rowcnt, H, N, CQ, fixq, st);
}
