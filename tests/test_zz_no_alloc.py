"""The allocation-free value-statistics entry point.

`t2t_vstats_gather_static` serves hosts that may not allocate device memory on
the request path: a process whose memory pool already owns the whole GPU, where
a late cudaMalloc fails or stalls.  It must give exactly what
`t2t_vstats_gather` gives with a caller-owned workspace, on back-to-back calls
(the built-in scratch keeps the previous call's contents), and must refuse
shapes beyond its fixed capacity without launching anything.  This file sorts
last so a run that stops at the first failure has already run everything else.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16
DEV = "cuda"


def _inputs(H, N, C, seed):
    g = torch.Generator().manual_seed(seed)
    v = torch.randn(H, N, 128, generator=g).to(BF)
    lab = torch.randint(0, C, (H, N), generator=g)
    lab[lab % 7 == 0] = 1                                   # some empty, one crowded cluster
    kperm = torch.sort(lab, dim=1, stable=True).indices.to(torch.int32)
    kcounts = torch.stack([torch.bincount(lab[h], minlength=C) for h in range(H)]).to(torch.int32)
    return v.to(DEV), kperm.to(DEV), kcounts.to(DEV)


def _outputs(H, N, C):
    return (torch.empty(H, N, 128, dtype=BF, device=DEV), torch.empty(H, C, 128, dtype=BF, device=DEV),
            torch.empty(H, dtype=torch.float32, device=DEV))


def test_static_scratch_variant_matches_workspace_variant_twice(lib):
    H, N, C = 2, 4096, 2048
    st = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(lib.t2t_vstats_gather_ws_bytes(H, C), dtype=torch.uint8, device=DEV)
    for seed in (21, 22):                                   # two calls in a row share the scratch
        v, kperm, kcounts = _inputs(H, N, C, seed)
        want = _outputs(H, N, C)
        got = _outputs(H, N, C)
        assert lib.t2t_vstats_gather(v.data_ptr(), kperm.data_ptr(), kcounts.data_ptr(), want[0].data_ptr(),
                                     want[1].data_ptr(), want[2].data_ptr(), H, N, C, ws.data_ptr(), ws.numel(),
                                     st) == 0
        assert lib.t2t_vstats_gather_static(v.data_ptr(), kperm.data_ptr(), kcounts.data_ptr(), got[0].data_ptr(),
                                            got[1].data_ptr(), got[2].data_ptr(), H, N, C, st) == 0
        torch.cuda.synchronize()
        assert torch.equal(got[0].view(torch.int16), want[0].view(torch.int16))
        assert torch.equal(got[1].view(torch.int16), want[1].view(torch.int16))
        assert torch.equal(got[2], want[2])


def test_static_scratch_variant_rejects_shapes_beyond_its_capacity(lib):
    cap = lib.t2t_vstats_gather_static_max_hc()
    assert cap == 8192
    H, N, C = 5, 4096, 2048                                  # 5 * 2048 > 8192
    v, kperm, kcounts = _inputs(1, N, C, 23)
    out = _outputs(1, N, C)
    st = torch.cuda.current_stream().cuda_stream
    rc = lib.t2t_vstats_gather_static(v.data_ptr(), kperm.data_ptr(), kcounts.data_ptr(), out[0].data_ptr(),
                                      out[1].data_ptr(), out[2].data_ptr(), H, N, C, st)
    assert rc == 4
    # the second limit: at most 4 heads, whatever the cluster count (8 * 1024 = 8192 clusters would fit the first)
    rc = lib.t2t_vstats_gather_static(v.data_ptr(), kperm.data_ptr(), kcounts.data_ptr(), out[0].data_ptr(),
                                      out[1].data_ptr(), out[2].data_ptr(), 8, N, 1024, st)
    assert rc == 4
    torch.cuda.synchronize()


def test_static_scratch_variant_at_exactly_its_capacity(lib):
    H, N, C = 4, 2048, 2048                                  # 4 heads x 2048 clusters: both limits met exactly
    st = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(lib.t2t_vstats_gather_ws_bytes(H, C), dtype=torch.uint8, device=DEV)
    v, kperm, kcounts = _inputs(H, N, C, 24)
    want, got = _outputs(H, N, C), _outputs(H, N, C)
    assert lib.t2t_vstats_gather(v.data_ptr(), kperm.data_ptr(), kcounts.data_ptr(), want[0].data_ptr(),
                                 want[1].data_ptr(), want[2].data_ptr(), H, N, C, ws.data_ptr(), ws.numel(), st) == 0
    assert lib.t2t_vstats_gather_static(v.data_ptr(), kperm.data_ptr(), kcounts.data_ptr(), got[0].data_ptr(),
                                        got[1].data_ptr(), got[2].data_ptr(), H, N, C, st) == 0
    torch.cuda.synchronize()
    for a, b in zip(got, want):
        assert torch.equal(a.view(torch.int16) if a.dtype == BF else a, b.view(torch.int16) if b.dtype == BF else b)
