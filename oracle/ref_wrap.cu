// C entry points around the reference's own launchers, so that the checker
// library oracle/_ref/libt2t_ref.so can be driven with ctypes.  The launchers
// themselves come from the reference checkout at build time (see build_ref.py);
// nothing of the reference is copied into this repository.  Test infrastructure
// only: the product never loads this library.
#include "kernels.h"   // kernels/kmeans_maintain/src
#include "kernel.h"    // kernels/select_union/src

extern "C" size_t ref_kmm_ws_bytes(int H, int N, int CQ, int CK) { return kmeans_maintain_ws_bytes(H, N, CQ, CK); }

extern "C" int ref_kmm_run(const void* QU, const void* KU, const void* V, const void* cq0, const void* ck0,
                           void* qlab, void* cq2, void* klab, void* ck2, void* qcounts, void* qperm,
                           void* kcounts, void* kperm, void* V_sorted, void* sumv, void* lam, int H, int N, int CQ,
                           int CK, int pin_tail, void* ws, void* stream) {
  kmeans_maintain_launch(QU, KU, V, cq0, ck0, qlab, cq2, klab, ck2, qcounts, qperm, kcounts, kperm, V_sorted,
                         sumv, lam, H, N, CQ, CK, pin_tail, ws, (cudaStream_t)stream);
  return (int)cudaGetLastError();
}

extern "C" size_t ref_vstats_ws_bytes(int H, int CK) { return reuse_vstats_ws_bytes(H, CK); }

extern "C" int ref_vstats_gather(const void* V, const void* kperm, const void* kcounts, void* V_sorted, void* sumv,
                                 void* lam, int H, int N, int CK, void* ws, void* stream) {
  reuse_vstats_gather_launch(V, kperm, kcounts, V_sorted, sumv, lam, H, N, CK, ws, (cudaStream_t)stream);
  return (int)cudaGetLastError();
}

extern "C" int ref_select_packed(const void* gl, const void* sizes, const void* rowlist, const void* tile_sizes,
                                 const void* ns, void* partial, void* packed, void* rowcnt, void* off, int H, int N,
                                 int CQ, void* stream) {
  fscu_packed_launch(gl, sizes, rowlist, tile_sizes, ns, partial, packed, rowcnt, off, H, N, CQ,
                     (cudaStream_t)stream);
  return (int)cudaGetLastError();
}
