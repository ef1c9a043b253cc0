/* C ABI of libt2t_b200.so: the Token2Tile sparse attention operator for B200
 * (sm_100a).
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, does
 * no allocation and no host synchronisation, and returns T2T_OK or an error
 * code after checking cudaGetLastError().  Workspaces are owned by the caller;
 * the *_ws_bytes functions give their sizes.  `d_status` (may be NULL) is a
 * device int that a kernel sets to a non-zero T2T_ST_* value when one of its
 * bounded waits gave up.
 *
 * Shapes use H heads, N tokens, D = 128, r = 32, C = 2048 key clusters and CQ
 * query clusters.  "bf16" tensors are row-major and contiguous.  Each function
 * names the reference interface it replaces by path:line inside the reference
 * project (token2tile/operator/...).
 */
#ifndef T2T_B200_H_
#define T2T_B200_H_

#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  T2T_OK = 0,
  T2T_ERR_ARG = 1,        /* null pointer, non-positive size, unsupported shape */
  T2T_ERR_CUDA = 2,       /* a launch or attribute call failed */
  T2T_ERR_WORKSPACE = 3,  /* workspace too small */
  T2T_ERR_TOO_LARGE = 4,  /* shape exceeds the fixed capacity of a no-allocation entry point */
};
enum {
  T2T_ST_OK = 0,
  T2T_ST_WAIT_TIMEOUT = 1,
  T2T_ST_BAD_PLAN = 2,
};

/* Library version as major * 10000 + minor * 100 + patch. */
int t2t_version(void);

/* out[h,n,:] = bf16(x[h,n,:] . U[h]) with fp32 accumulation on the tensor
 * cores.  x bf16 [H,N,128], U bf16 [H,128,32], out bf16 [H,N,32].
 * Replaces torch.bmm(q, Uq, out=QU) / torch.bmm(k, Uk, out=KU),
 * deploy_step.py:321-324 and :252-253. */
int t2t_project(const void* x, const void* U, void* out, int H, int N, int* d_status,
                cudaStream_t stream);

/* Projection fit: fp32 Uq, Uk [H,128,32] minimising ||Q K^T - (Q Uq)(K Uk)^T||_F
 * for q, k bf16 [H,N,128].  Second moments on the tensor cores (fp32 slabs of
 * 8192 rows, summed in fp64 in slab order), symmetric roots and singular
 * triplets by an fp64 Jacobi kernel (one CTA per matrix, eigenvalues clamped
 * at 1e-8), all batched over heads on `stream` without a host round trip.
 * d_bad: int [2 H], set to 1 for a head whose q (first H) or k (last H) holds a
 * non-finite value; that head's Uq, Uk are left untouched.  ws:
 * t2t_lowrank_fit_ws_bytes(H, N).  Replaces online_u, deploy_step.py:122-149
 * (and its batched forms, integrations/sglang/backend/t2t_attn.py:181-239). */
size_t t2t_lowrank_fit_ws_bytes(int H, int N);
int t2t_lowrank_fit(const void* q, const void* k, float* Uq, float* Uk, int H, int N, void* ws,
                    size_t ws_bytes, int* d_bad, int* d_status, cudaStream_t stream);

/* labels[h,i] = argmin_c(||c||^2 - 2 x_i.c), ties to the lowest c; rows >=
 * pin_begin get pin_label when pin_begin >= 0.  x bf16 [H,N,32], cen bf16
 * [H,Cn,32], labels int32 [H,N].  The distance is DEFINED as the fp32
 * fused-multiply-add chain over k = 0..31 started at ||c||^2, so labels are
 * reproducible bit for bit on any machine.  t2t_assign finds them with a
 * tcgen05 product and re-evaluates by the exact chain only the rows whose two
 * nearest centroids are closer than the product's error bound;
 * t2t_assign_exact evaluates the chain for every pair (slow; the cross-check).
 * Both give identical labels.  ws: t2t_assign_ws_bytes(H, N).  Replaces
 * fast_assign(x, centroids), fast_assign.py:79-106 and assign_kernel,
 * kernels/kmeans_maintain/src/kernels.cu:104-257. */
size_t t2t_assign_ws_bytes(int H, int N);
int t2t_assign(const void* x, const void* cen, void* labels, int H, int N, int Cn, int pin_begin,
               int pin_label, void* ws, size_t ws_bytes, int* d_status, cudaStream_t stream);
int t2t_assign_exact(const void* x, const void* cen, void* labels, int H, int N, int Cn, int pin_begin,
                     int pin_label, cudaStream_t stream);

/* Deterministic centroid update from labels: integer fixed-point (2^15) sums,
 * newc = bf16(float(sum) / (2^15 n)), an empty cluster keeps `old`.  x bf16
 * [H,N,32], labels int32 [H,N], old/newc bf16 [H,Cn,32], counts int32 [H,Cn].
 * Replaces fused_update_vstats(ku, labels, old, None),
 * fused_update_vstats.py:72-115 (its deterministic form,
 * integrations/sglang/backend/t2t_attn.py:242-257). */
size_t t2t_centroid_update_ws_bytes(int H, int N, int Cn);
int t2t_centroid_update(const void* x, const void* labels, const void* old, void* newc, void* counts,
                        int H, int N, int Cn, void* ws, size_t ws_bytes, cudaStream_t stream);

/* One structure rebuild: two Lloyd passes for the queries (from cq0), one for
 * the keys (from ck0), stable grouping of both, fp32 key means, cluster-major
 * V and the per-cluster value sums.  Outputs: qlab/klab int32 [H,N], cq2 bf16
 * [H,CQ,32], ck2 fp32 [H,C,32], ck16 = bf16(ck2), cks16 = bf16(ck2 * scale),
 * qcounts int32 [H,CQ], qperm/kperm int32 [H,N] (sorted position -> row),
 * kcounts int32 [H,C], V_sorted bf16 [H,N,128], sumv bf16 [H,C,128] (value sums
 * divided by lam), lam fp32 [H].  The last pin_tail keys are forced into
 * cluster C-1.  Replaces kmeans_maintain_launch,
 * kernels/kmeans_maintain/src/kernels.h:5-13 (kernels.cu:787-876) and the casts
 * at deploy_step.py:389-393.  The key side runs on a stream the library creates
 * once per device, forked from `stream` by an event and joined back before the
 * call returns: the caller sees one call ordered on its stream. */
size_t t2t_kmeans_maintain_ws_bytes(int H, int N, int CQ, int C);
int t2t_kmeans_maintain(const void* QU, const void* KU, const void* V, const void* cq0, const void* ck0,
                        void* qlab, void* cq2, void* klab, void* ck2, void* ck16, void* cks16,
                        void* qcounts, void* qperm, void* kcounts, void* kperm, void* V_sorted,
                        void* sumv, void* lam, float scale, int H, int N, int CQ, int C, int pin_tail,
                        void* ws, size_t ws_bytes, int* d_status, cudaStream_t stream);

/* Reuse call: V_sorted = V[kperm], value sums and lam from this call's V with
 * the stored grouping.  Replaces reuse_vstats_gather_launch,
 * kernels/kmeans_maintain/src/kernels.h:22-26 (kernels.cu:900-923). */
size_t t2t_vstats_gather_ws_bytes(int H, int C);
int t2t_vstats_gather(const void* V, const void* kperm, const void* kcounts, void* V_sorted, void* sumv,
                      void* lam, int H, int N, int C, void* ws, size_t ws_bytes, cudaStream_t stream);

/* t2t_vstats_gather for callers that cannot allocate device memory.  It has no
 * counterpart in the reference.  Some hosts hand the whole device to their own
 * memory pool when they start (serving engines that pre-size their caches), or
 * run under a policy that forbids driver allocations on the request path
 * because cudaMalloc can fail late or stall the device; such a caller has no
 * workspace to pass.  This variant takes none: its scratch is a fixed array
 * inside the library image, T2T_STATIC_VSTATS_MAX_HC * 516 bytes (about 4 MB)
 * resident on every GPU that loads the library, for as long as the process
 * lives.  Inputs and outputs are still the caller's.  Limits and rules:
 *   - two limits, both checked before anything is launched: H must not exceed
 *     T2T_STATIC_VSTATS_MAX_HC / 2048 = 4 heads (the per-head block maxima
 *     have room for that many), and H * C must not exceed
 *     T2T_STATIC_VSTATS_MAX_HC (so 4 heads of 2048 clusters fit, 8 heads of
 *     1024 do not); anything larger returns T2T_ERR_TOO_LARGE;
 *   - the first call on each device looks up the array's device address (with
 *     that device current); make that first call outside any stream capture;
 *   - all calls share the one array and it keeps the last call's contents; the
 *     kernels overwrite every word before reading it, so nothing is cleared,
 *     but two calls that overlap on the GPU (different streams) race;
 *   - it calls no cudaMalloc, cudaFree or allocating library routine. */
#define T2T_STATIC_VSTATS_MAX_HC 8192
size_t t2t_vstats_gather_static_max_hc(void);
int t2t_vstats_gather_static(const void* V, const void* kperm, const void* kcounts, void* V_sorted, void* sumv,
                             void* lam, int H, int N, int C, cudaStream_t stream);

/* out[h,i,:] = x[h,perm[h,i],:] for rows of 128 bf16.  Replaces
 * fast_gather(x, perm, out), fast_permute.py:54-56. */
int t2t_gather_rows(const void* x, const void* perm, void* out, int H, int N, cudaStream_t stream);

/* Scoring and selection fused: g = fp16(QU_i . cks_c) (DEFINED as the fp32
 * fused-multiply-add chain over k), clusters ordered by (g descending, index
 * ascending), a cluster is selected iff the sizes before it sum to < *ns; the
 * selections of a query cluster are OR-ed into unip int32 [H,CQ,64] (bit b of
 * word w = cluster 32 w + b); rowcnt int32 [H,N] is the selected token count per
 * query.  qperm/tile_sizes are the query grouping; ns is a device int32 read by
 * the kernel (N < 2^19); pin_tail > 0 also sets cluster C-1 in every row.  The
 * [H,N,2048] score matrix is never stored.  t2t_score_select_union scores on
 * the tensor cores and settles each row from the approximate scores plus exact
 * chain scores of the few clusters near its threshold; rows it cannot settle
 * that way go to the exact routine.  t2t_score_select_union_exact evaluates
 * every chain (slow; the cross-check).  Both give identical results.  ws:
 * t2t_score_select_union_ws_bytes(H, N).  Replaces torch.bmm(QU, cks^T, out=gl),
 * deploy_step.py:394, fscu_packed_launch / fscu_split_packed_launch,
 * kernels/select_union/src/kernel.h:19-29 (kernel.cu:523-556), and the pin_tail
 * OR at deploy_step.py:444-448. */
size_t t2t_score_select_union_ws_bytes(int H, int N);
int t2t_score_select_union(const void* QU, const void* cks, const void* kcounts, const void* qperm,
                           const void* tile_sizes, const int* ns, void* unip, void* rowcnt, int H,
                           int N, int CQ, int pin_tail, void* ws, size_t ws_bytes, int* d_status,
                           cudaStream_t stream);
int t2t_score_select_union_exact(const void* QU, const void* cks, const void* kcounts, const void* qperm,
                                 const void* tile_sizes, const int* ns, void* unip, void* rowcnt, int H,
                                 int N, int CQ, int pin_tail, cudaStream_t stream);

/* Task plan + exact attention over the unions + centroid residual + merge.
 * q bf16 [H,N,128] original order; kp/vp bf16 [H,N,128] cluster-major;
 * tile_sizes int32 [H,CQ]; kcounts int32 [H,C]; unip int32 [H,CQ,64]; QU bf16
 * [H,N,32]; cks bf16 [H,C,32]; sumv bf16 [H,C,128]; lam fp32 [H]; qlab, qperm
 * int32 [H,N]; tailw device fp32; out bf16 [H,N,128] original order.  plan
 * (t2t_tile_attn_plan_ints ints) belongs to the structure snapshot and is
 * rebuilt when rebuild_plan != 0; ws (t2t_tile_attn_ws_bytes) holds the
 * intermediate exact output and log-sum-exp.  Replaces launch_cluster_attn +
 * launch_tail_merge, kernels/tile_attn/src/main.cpp:5-14, 24-50 and
 * plan_workspace_ints, main.cpp:16-22. */
size_t t2t_tile_attn_plan_ints(int H, int N, int CQ);
size_t t2t_tile_attn_ws_bytes(int H, int N);
int t2t_tile_attn(const void* q, const void* kp, const void* vp, const void* tile_sizes,
                  const void* kcounts, const void* unip, const void* QU, const void* cks,
                  const void* sumv, const void* lam, const void* qlab, const void* qperm,
                  const float* tailw, void* out, int* plan, int rebuild_plan, int H, int N, int CQ,
                  void* ws, size_t ws_bytes, int* d_status, cudaStream_t stream);

/* The three stages of t2t_tile_attn as separate calls (same arguments), so a
 * caller can time or overlap them: the task plan (kv lengths, key-cluster
 * offsets, tasks in longest-first order; selected_kv_lengths_kernel and
 * plan_kernel, kernels/tile_attn/src/kernel.cu:259-378), the exact attention
 * over the unions (attn_kernel, kernel.cu:820-1096) and the residual + merge
 * (tail_wgmma_kernel, kernel.cu:1172-1450). */
int t2t_tile_attn_plan(const void* tile_sizes, const void* kcounts, const void* unip, int* plan, int H, int N,
                       int CQ, cudaStream_t stream);
int t2t_tile_attn_exact(const void* q, const void* kp, const void* vp, const void* unip, const void* qperm,
                        int* plan, int H, int N, int CQ, void* ws, size_t ws_bytes, int* d_status,
                        cudaStream_t stream);
int t2t_tile_attn_merge(const void* QU, const void* cks, const void* sumv, const void* kcounts, const void* unip,
                        const void* qlab, const void* qperm, const void* lam, const float* tailw, void* out,
                        int H, int N, int CQ, void* ws, size_t ws_bytes, int* d_status, cudaStream_t stream);

/* Number of tasks and executed (query, key) pairs of the current plan, for
 * FLOP accounting: info[0] = tasks, info[1..2] = pairs as low/high 32 bits.
 * Device-side; copies 4 ints into d_info. */
int t2t_tile_attn_plan_info(const int* plan, int H, int N, int CQ, int* d_info, cudaStream_t stream);

/* The same entry points for q, k, v (and the output) given as VIEWS of a tensor laid out [N, H, 128], the way
 * the reference's serving host holds them (integrations/sglang/backend/t2t_attn.py:1160-1163, where the
 * reference pays three transposing copies in and one out).  Row (h, n) of such a tensor starts at
 * base + h * head_stride + n * row_stride (strides in ELEMENTS; 128 and N * 128 for the contiguous [H, N, 128]
 * layout; 128 * H and 128 for a [N, H, 128] tensor).  Both strides must be multiples of 128 where a tensor
 * feeds a TMA row gather (q of the attention, out of the merge) and of 8 elsewhere; the 128 elements of a row
 * are contiguous.  Everything else is as in the entry points without the suffix, which forward here. */
int t2t_project_strided(const void* x, long long x_row_stride, long long x_head_stride, const void* U, void* out,
                        int H, int N, int* d_status, cudaStream_t stream);
int t2t_lowrank_fit_strided(const void* q, const void* k, long long row_stride, long long head_stride, float* Uq,
                            float* Uk, int H, int N, void* ws, size_t ws_bytes, int* d_bad, int* d_status,
                            cudaStream_t stream);
int t2t_gather_rows_strided(const void* x, long long x_row_stride, long long x_head_stride, const void* perm,
                            void* out, int H, int N, cudaStream_t stream);
int t2t_kmeans_maintain_strided(const void* QU, const void* KU, const void* V, long long v_row_stride,
                                long long v_head_stride, const void* cq0, const void* ck0, void* qlab, void* cq2,
                                void* klab, void* ck2, void* ck16, void* cks16, void* qcounts, void* qperm,
                                void* kcounts, void* kperm, void* V_sorted, void* sumv, void* lam, float scale,
                                int H, int N, int CQ, int C, int pin_tail, void* ws, size_t ws_bytes,
                                int* d_status, cudaStream_t stream);
int t2t_vstats_gather_strided(const void* V, long long v_row_stride, long long v_head_stride, const void* kperm,
                              const void* kcounts, void* V_sorted, void* sumv, void* lam, int H, int N, int C,
                              void* ws, size_t ws_bytes, cudaStream_t stream);
int t2t_tile_attn_exact_strided(const void* q, long long q_row_stride, long long q_head_stride, const void* kp,
                                const void* vp, const void* unip, const void* qperm, int* plan, int H, int N,
                                int CQ, void* ws, size_t ws_bytes, int* d_status, cudaStream_t stream);
int t2t_tile_attn_merge_strided(const void* QU, const void* cks, const void* sumv, const void* kcounts,
                                const void* unip, const void* qlab, const void* qperm, const void* lam,
                                const float* tailw, void* out, long long out_row_stride, long long out_head_stride,
                                int H, int N, int CQ, void* ws, size_t ws_bytes, int* d_status,
                                cudaStream_t stream);

/* Tensor-core self-test: S = A . B^T, O = bf16(S / 16) . V for 128 x 128 bf16
 * operands, through the same shared-memory / TMEM operand forms the attention
 * kernels use.  No counterpart in the reference. */
int t2t_umma_selftest(const void* A, const void* B, const void* V, float* S_out, float* O_out,
                      int* d_status, cudaStream_t stream);

/* TMA row-gather self-test: gathers the 128 rows `gidx[0..127]` of the bf16
 * matrix src [rows, 128] into one SWIZZLE_128B shared-memory tile (two blocks of
 * 64 columns, 128-byte rows, 16-byte chunk c of row r stored at chunk
 * c ^ (r & 7)) and copies the tile's 32 KB to `out` unchanged.  Same tensor map
 * and instruction form as the attention kernel's K / V tile loads.  No
 * counterpart in the reference. */
int t2t_gather4_selftest(const void* src, int rows, const int* gidx, void* out, int* d_status,
                         cudaStream_t stream);

/* Bounded-wait self-test: one CTA waits on a barrier that nothing arrives on, with a
 * spin limit of about a millisecond, and leaves the way the production kernels do when
 * a wait gives up: *d_status becomes 1 (wait timed out), d_out[0..1] = 0 (both warps'
 * waits returned "gave up": the first by its limit, the second by the abort flag).  The
 * kernel always terminates.  No counterpart in the reference. */
int t2t_wait_timeout_selftest(int* d_status, int* d_out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* T2T_B200_H_ */
