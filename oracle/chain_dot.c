/* CPU oracle helper (test infrastructure only): the ordered fp32 chain that
 * defines every integer decision of the operator,
 *
 *     out[i][j] = fl32(... fl32(fl32(init[j] + x[i][0] c[j][0]) + x[i][1] c[j][1]) ... ),
 *
 * k = 0 .. r-1 in order, each product and each sum rounded to fp32 separately
 * (compiled with -ffp-contract=off; for 16-bit inputs the products are exact, so a
 * fused multiply-add chain gives the same bits).  It restates the arithmetic the
 * reference's kernels apply per (row, centroid) pair
 * (kernels/kmeans_maintain/src/kernels.cu:102-257, kernels/select_union/src/kernel.cu:190-260
 * up to the accumulation order, which this build fixes to index order) and is a
 * faster twin of t2t_oracle.chain_dot's PyTorch loop: same bits, checked in
 * tests/test_oracle_cpu.py.  Rows are independent and run on all host threads. */
#include <stdlib.h>
#include <string.h>

int t2t_chain_dot(const float* x, const float* c, const float* init, float* out, long n, long m, int r) {
  if (n < 0 || m <= 0 || r <= 0) return 1;
  float* ct = (float*)malloc((size_t)r * (size_t)m * sizeof(float));   /* c transposed: [k][j] */
  if (!ct) return 2;
  for (long j = 0; j < m; ++j)
    for (int k = 0; k < r; ++k) ct[(size_t)k * m + j] = c[(size_t)j * r + k];
#pragma omp parallel for schedule(static)
  for (long i = 0; i < n; ++i) {
    float* o = out + (size_t)i * m;
    if (init) memcpy(o, init, (size_t)m * sizeof(float));
    else memset(o, 0, (size_t)m * sizeof(float));
    for (int k = 0; k < r; ++k) {
      const float xv = x[(size_t)i * r + k];
      const float* row = ct + (size_t)k * m;
      for (long j = 0; j < m; ++j) {
        const float p = xv * row[j];
        o[j] = o[j] + p;
      }
    }
  }
  free(ct);
  return 0;
}
