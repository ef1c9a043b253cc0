#!/usr/bin/env python
"""Benchmark of the Token2Tile attention layer on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N ...

Metric: milliseconds per attention layer at the Wan2.1-14B 720p shape
(75,600 tokens x 40 heads x 128, bf16, 1.5 % budget, 512 query clusters).  A
step is one full (structure-rebuilding) call of the layer; reuse calls and the
1-rebuild-in-8 amortised figure are reported beside it.  With N GPUs the 40
heads are split N ways (no traffic inside the operator); the value is the
maximum over ranks, i.e. the whole-box time of the layer.

Inputs are seeded synthetic tensors (token2tile_b200/synth.py); 2.3 GB of
q/k/v per step is far larger than L2, so no flush is needed between steps.
`--impl reference` times the CPU restatement of the operator (oracle/) on the
host cores for one head per step and scales to 40 heads.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOAD = dict(name="wan2.1-14b-720p-self-attention-layer", H=40, grid="720p", N=75600, CQ=512, D=128,
                s_frac=0.015)
KERNELS_REBUILD = 2 + 21 + 3 + 1 + 1 + 3  # project, kmeans (3 assign+fix, 3x3 grouping, 3 means, 3 value stats), centroid moments+select+fix, gather, plan, attention (two kernels) + merge
KERNELS_REUSE = 1 + 1 + 3 + 3   # project q, gather k, value stats, attention (two kernels) + merge
ATTN_DRAM_BYTES_480P_8H = 444.2e6      # attn2_kernel (206.6 MB) + attn_kernel (210.9 MB), H 8, N 32,760 (ncu)
METRIC = "t2t_attn_ms_per_layer"
UNIT = "ms/layer"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf=1400.0, src="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "100", "-i", str(index)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        if self.p is None:
            return None
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        rows = [r.split(",") for r in Path(self.f.name).read_text().strip().splitlines() if r.count(",") >= 6]
        os.unlink(self.f.name)
        if not rows:
            return None
        try:
            sm = sorted(float(r[0]) for r in rows)
            reasons = []
            for i, name in ((3, "hw_slowdown"), (4, "hw_thermal_slowdown"), (5, "sw_thermal_slowdown"),
                            (6, "sw_power_cap")):
                if any("Active" in r[i] and "Not" not in r[i] for r in rows):
                    reasons.append(name)
            return dict(sm_mhz=sm[len(sm) // 2], sm_max_mhz=float(rows[0][1]), samples=len(rows),
                        power_w_max=max(float(r[2]) for r in rows), reasons=reasons)
        except ValueError:
            return None


def time_events(fn, steps, stream=None):
    """Device time of `steps` calls of fn, in ms, by CUDA events on the current stream."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1)


def dense_attention_ms(q, k, v, warm=3, timed=10):
    """Fastest dense attention on this box for the same tensors: per library the
    median of `timed` calls (each timed on its own by CUDA events) after `warm`
    warm-ups."""
    import torch.nn.functional as F
    out = {}
    qb, kb, vb = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
    cands = {}
    try:
        from torch.nn.attention import SDPBackend, sdpa_kernel
        for name, be in (("sdpa_flash", SDPBackend.FLASH_ATTENTION), ("sdpa_cudnn", SDPBackend.CUDNN_ATTENTION)):
            def run(be=be):
                with sdpa_kernel([be]):
                    return F.scaled_dot_product_attention(qb, kb, vb)
            cands[name] = run
    except ImportError:
        pass
    try:
        from flash_attn import flash_attn_func
        qf, kf, vf = (t.transpose(0, 1).unsqueeze(0).contiguous() for t in (q, k, v))
        cands["flash_attn"] = lambda: flash_attn_func(qf, kf, vf)
    except Exception:      # noqa: BLE001 - optional library
        pass
    try:
        import flashinfer
        qi, ki, vi = (t.transpose(0, 1).contiguous() for t in (q, k, v))
        cands["flashinfer"] = lambda: flashinfer.single_prefill_with_kv_cache(qi, ki, vi, causal=False)
    except Exception:      # noqa: BLE001 - optional library
        pass
    for name, run in cands.items():
        try:
            for _ in range(warm):
                run()
            ts = sorted(time_events(run, 1) for _ in range(timed))
            out[name] = ts[len(ts) // 2]
        except Exception as exc:      # noqa: BLE001 - a backend may refuse the shape
            out[name] = None
            print(f"[bench] dense backend {name} unavailable: {type(exc).__name__}", file=sys.stderr)
    return out


# ---------------------------------------------------------------------------
# CPU arm: the oracle on the host cores, one head per step
# ---------------------------------------------------------------------------

def cpu_head_step_factory(seed_head=0):
    from oracle import t2t_oracle as O
    from token2tile_b200.synth import GRIDS, locality_mixture
    O.FAST_DOT = True          # sgemm instead of the bit-exact chain: this leg is timed, not compared
    W = WORKLOAD
    torch.set_num_threads(os.cpu_count() or 1)
    q, k, v = locality_mixture(1, GRIDS[W["grid"]], heads=[seed_head])
    op = O.OracleOperator(1, W["N"], W["CQ"], s_frac=W["s_frac"])
    state = op.init_state(q, k, warm_iters=1)

    def step():
        st = dict(state)
        t0 = time.perf_counter()
        op.step(q, k, v, st)
        return (time.perf_counter() - t0) * 1e3 * W["H"]      # one head, scaled to the 40-head layer
    return step, torch.get_num_threads()


def cpu_small_config():
    """The reference's CPU-runnable configuration on the host cores: one init_state and one rebuild call of
    the oracle operator, and dense fp32 attention at the same shape."""
    from oracle import t2t_oracle as O
    from token2tile_b200.synth import GRIDS, locality_mixture
    O.FAST_DOT = True
    H, N, CQ = 2, 4096, 32
    q, k, v = locality_mixture(H, GRIDS["cpu"], dtype=torch.float32)
    op = O.OracleOperator(H, N, CQ, s_frac=0.05, dtype=torch.float32)
    t0 = time.perf_counter()
    state = op.init_state(q, k)
    t1 = time.perf_counter()
    op.step(q, k, v, state)
    t2 = time.perf_counter()
    torch.nn.functional.scaled_dot_product_attention(q, k, v)
    t3 = time.perf_counter()
    return {"shape": "H 2, N 4096, CQ 32, fp32, 5 % budget", "init_state_ms": (t1 - t0) * 1e3,
            "rebuild_step_ms": (t2 - t1) * 1e3, "dense_fp32_ms": (t3 - t2) * 1e3}


def run_reference(args, rank):
    if rank != 0:
        return
    step, cores = cpu_head_step_factory()
    for _ in range(args.warmup):
        step()
    ts = [step() for _ in range(args.steps)]
    val = sum(ts) / len(ts)
    sample = "one head of 40 per step (full 75,600 tokens), time x 40"
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": val, "higher_is_better": False,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD["name"], **{k: WORKLOAD[k] for k in ("H", "N", "CQ", "D", "s_frac")}},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ---------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------

def layer_480p(dev, lo, hi, maxr, barrier):
    """The 480p layer (N 32,760, CQ 256) for this rank's heads: rebuild and reuse call times at the 1.5 % and
    5 % budgets, the fastest dense attention on the same tensors and the relative L2 distance from it."""
    from token2tile_b200 import MaskedStepDeploy
    from token2tile_b200.synth import GRIDS, locality_mixture
    import torch.nn.functional as F
    N, CQ = 32760, 256
    q, k, v = (t.to(dev) for t in locality_mixture(hi - lo, GRIDS["480p"], heads=range(lo, hi)))
    dense = dense_attention_ms(q, k, v, warm=2, timed=5)
    dense_ok = [t for t in dense.values() if t]
    dense_best = maxr(min(dense_ok)) if dense_ok else None
    dense_out = F.scaled_dot_product_attention(q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0))[0].float()
    out = {"N": N, "CQ": CQ, "heads_per_gpu": hi - lo, "dense_ms": dense, "fastest_dense_ms": dense_best, "budgets": {}}
    for frac in (0.015, 0.05):
        op = MaskedStepDeploy(hi - lo, N, CQ, s_frac=frac, device=dev, mask_refresh=4)
        state = op.init_state(q, k, warm_iters=4, seed=0)

        clock = [0]

        def rebuild():
            clock[0] += 4                          # a refresh period later: branch 0 rebuilds
            op.set_cfg_call(0, key=0, step=clock[0])
            op.step(q, k, v, state)

        def reuse():
            op.set_cfg_call(1, key=0, step=clock[0])
            op.step(q, k, v, state)

        for _ in range(3):
            rebuild()
        barrier()
        rb = maxr(time_events(rebuild, 5) / 5)
        assert op.last_rebuilt is True
        clock[0] += 4
        op.set_cfg_call(0, key=0, step=clock[0])
        res = op.step(q, k, v, state).float()
        rel = float(((res - dense_out).norm() / dense_out.norm()).item())
        reuse()
        barrier()
        ru = maxr(time_events(reuse, 5) / 5)
        assert op.last_rebuilt is False and op.device_status() == 0
        amort = (rb + 7 * ru) / 8
        out["budgets"][f"{frac * 100:g}%"] = {
            "ns": op.ns, "rebuild_ms": rb, "reuse_ms": ru, "amortised_ms_1_rebuild_7_reuse": amort,
            "rel_l2_vs_dense": maxr(rel),
            "speedup_vs_dense": {"rebuild": dense_best / rb, "reuse": dense_best / ru, "amortised": dense_best / amort}
            if dense_best else None}
        del op, state, res
    return out


def run_ours(args, rank, world, local_rank):
    from token2tile_b200 import MaskedStepDeploy
    from token2tile_b200.parallel import head_range
    from token2tile_b200.synth import GRIDS, locality_mixture
    import torch.distributed as dist

    W = dict(WORKLOAD)
    if args.heads or args.grid:      # smaller cases for profiler captures; the default is the 720p layer
        W["H"] = args.heads or W["H"]
        W["grid"] = args.grid or W["grid"]
        W["N"] = GRIDS[W["grid"]][0] * GRIDS[W["grid"]][1] * GRIDS[W["grid"]][2]
        W["CQ"] = {"720p": 512, "480p": 256, "cpu": 32}[W["grid"]]
        W["name"] = f"self-attention-layer-{W['grid']}-{W['H']}heads"
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lo, hi = head_range(rank, world, W["H"])
    Hl, N, CQ = hi - lo, W["N"], W["CQ"]
    q, k, v = locality_mixture(Hl, GRIDS[W["grid"]], heads=range(lo, hi))
    hq, hk, hv = q.pin_memory(), k.pin_memory(), v.pin_memory()
    qd, kd, vd = hq.to(dev), hk.to(dev), hv.to(dev)
    hout = torch.empty(Hl, N, W["D"], dtype=torch.bfloat16).pin_memory()

    op = MaskedStepDeploy(Hl, N, CQ, s_frac=W["s_frac"], device=dev, mask_refresh=1)
    state0 = op.init_state(qd, kd, warm_iters=4, seed=0)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def maxr(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    state = dict(state0)

    def rebuild_step():
        op.step(qd, kd, vd, state)

    for _ in range(args.warmup):
        rebuild_step()
    barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms = time_events(rebuild_step, args.steps)
    barrier()
    clocks = sampler.stop() if sampler else None
    ms_step = maxr(ms / args.steps)
    assert op.device_status() == 0, "a device wait timed out"

    # per-stage device times of one rebuild call
    op.profile = True
    rebuild_step()
    stages = op.stage_times()
    op.profile = False
    tasks, pairs = op.plan_info()
    # rows of the query clusters against the 128-row tensor-core tiles their tasks occupy: full 256-row tasks and
    # remainders above 128 rows take two tiles, remainders of at most 128 rows one
    sizes = op.last_structure["tile_sizes"].to(torch.int64)
    rem = sizes % 256
    row_tiles = 2 * (sizes // 256) + (rem > 128).to(torch.int64) * 2 + ((rem > 0) & (rem <= 128)).to(torch.int64)
    m_util = float(sizes.sum().item()) / max(1.0, 128.0 * float(row_tiles.sum().item()))
    if args.light:
        if rank == 0:
            print(json.dumps({"metric": METRIC, "value": ms_step, "unit": UNIT, "n_gpus": world,
                              "config": {"workload": W["name"], "H": W["H"], "N": N, "CQ": CQ},
                              "stages_ms": stages, "tasks": tasks, "pairs": pairs, "m_utilisation": m_util,
                              "clocks": clocks}))
        if world > 1:
            dist.destroy_process_group()
        return

    # end to end: host buffers in, host buffer out, through the same call
    def e2e_step():
        qd.copy_(hq, non_blocking=True)
        kd.copy_(hk, non_blocking=True)
        vd.copy_(hv, non_blocking=True)
        out = op.step(qd, kd, vd, state)
        hout.copy_(out, non_blocking=True)

    e2e_step()
    barrier()
    e2e_serial_ms = maxr(time_events(e2e_step, max(2, args.steps // 2)) / max(2, args.steps // 2))
    barrier()

    # The same with double-buffered inputs and outputs, the way a serving loop feeds the operator: the copies
    # of step i + 1 run on a copy stream while step i computes, the result of step i leaves on a third stream
    # while step i + 1 computes into the other output tensor.  Every step still copies its own q, k, v in and
    # its own output out inside the timed region, which also contains the fill and the drain of the pipeline.
    s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    in_bufs = [(qd, kd, vd), tuple(torch.empty_like(t) for t in (qd, kd, vd))]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_free = [torch.cuda.Event() for _ in range(2)]
    ev_comp = torch.cuda.Event()
    ev_out = [torch.cuda.Event() for _ in range(2)]
    out_bufs = [torch.empty_like(op.tile_attn_out) for _ in range(2)]

    def e2e_pipelined(nsteps):
        cur = torch.cuda.current_stream(dev)
        for e in ev_free + ev_out:
            e.record(cur)
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        for i in range(nsteps + 1):
            if i < nsteps:
                b = i & 1
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_free[b])            # the step that read this buffer has finished
                    for dst, src in zip(in_bufs[b], (hq, hk, hv)):
                        dst.copy_(src, non_blocking=True)
                    ev_in[b].record(s_in)
            if i >= 1:
                b = (i - 1) & 1
                cur.wait_event(ev_in[b])
                cur.wait_event(ev_out[b])                  # the result before last has left this output tensor
                out = op.step(*in_bufs[b], state, out=out_bufs[b])
                ev_free[b].record(cur)
                ev_comp.record(cur)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_comp)
                    hout.copy_(out, non_blocking=True)
                    ev_out[b].record(s_out)
        for e in ev_out:
            cur.wait_event(e)

    e2e_pipelined(2)
    barrier()
    n_e2e = max(8, args.steps)
    e2e_ms = maxr(time_events(lambda: e2e_pipelined(n_e2e), 1) / n_e2e)
    barrier()
    del in_bufs, out_bufs

    # reuse calls (structure held, values recomputed)
    opr = op
    opr.mask_refresh, opr._cfg_on = 4, True
    opr.set_cfg_call(0, key=0, step=0)
    opr.step(qd, kd, vd, state)
    cnt = [0]

    def reuse_step():
        cnt[0] += 1
        opr.set_cfg_call(1, key=0, step=0)
        opr.step(qd, kd, vd, state)

    reuse_step()
    barrier()
    reuse_ms = maxr(time_events(reuse_step, max(2, args.steps // 2)) / max(2, args.steps // 2))
    assert opr.last_rebuilt is False
    op.profile = True
    reuse_step()
    reuse_stages = op.stage_times()
    op.profile = False
    barrier()

    dense = dense_attention_ms(qd, kd, vd)
    dense_ok = {n: t for n, t in dense.items() if t}
    dense_best = maxr(min(dense_ok.values())) if dense_ok else None

    # budgets of the layer (1.25 %, 1.5 %, 5 % of the tokens per query): rebuild time and the relative L2
    # distance of the output from dense attention on the same tensors
    import torch.nn.functional as F
    budgets = {}
    try:
        dense_out = F.scaled_dot_product_attention(qd.unsqueeze(0), kd.unsqueeze(0), vd.unsqueeze(0))[0].float()
        dn = dense_out.norm()
        ns_keep = int(op.ns_t.item())
        op.mask_refresh, op._cfg_on = 1, False
        for frac in (0.0125, 0.015, 0.05):
            op.ns_t.fill_(max(1, int(frac * N)))
            st_b = dict(state0)
            op.step(qd, kd, vd, st_b)
            ms_b = maxr(time_events(lambda: op.step(qd, kd, vd, st_b), 3) / 3)
            rel = float(((op.step(qd, kd, vd, st_b).float() - dense_out).norm() / dn).item())
            budgets[f"{frac * 100:g}%"] = {"ns": int(op.ns_t.item()), "rebuild_ms": ms_b, "rel_l2_vs_dense": maxr(rel)}
        op.ns_t.fill_(ns_keep)
        del dense_out
    except Exception as exc:      # noqa: BLE001 - the comparison is informative, not part of the metric
        print(f"[bench] budget sweep skipped: {type(exc).__name__}: {exc}", file=sys.stderr)

    # state initialisation (once per request, layer and branch): the operator's own and the fast variant
    init_ms = {}
    try:
        from token2tile_b200 import t2t_attn as B
        t0 = time.perf_counter(); op.init_state(qd, kd, warm_iters=4, seed=0); torch.cuda.synchronize()
        init_ms["init_state"] = maxr((time.perf_counter() - t0) * 1e3)
        fast = B.make_fast_init_state(op)
        fast(qd, kd, warm_iters=4, seed=0); torch.cuda.synchronize()
        t0 = time.perf_counter(); fast(qd, kd, warm_iters=4, seed=0); torch.cuda.synchronize()
        init_ms["fast_init_state"] = maxr((time.perf_counter() - t0) * 1e3)
    except Exception as exc:      # noqa: BLE001
        print(f"[bench] init timing skipped: {type(exc).__name__}: {exc}", file=sys.stderr)

    ns_layer = op.ns
    # BASELINE configuration 2: the 480p layer (32,760 tokens, 256 query clusters), budgets 1.5 % and 5 %
    config2 = None
    if not (args.heads or args.grid):
        try:
            del qd, kd, vd, hq, hk, hv, hout
            torch.cuda.empty_cache()
            config2 = layer_480p(dev, lo, hi, maxr, barrier)
        except Exception as exc:      # noqa: BLE001 - a second, informative measurement
            print(f"[bench] 480p configuration skipped: {type(exc).__name__}: {exc}", file=sys.stderr)

    # BASELINE configuration 5 at eight GPUs: the full transformer step (40 blocks, Ulysses x8) with Token2Tile
    # and with dense self-attention, one refresh period each
    dit = None
    if world == 8 and not (args.heads or args.grid):
        try:
            del op, opr, state, state0
            torch.cuda.empty_cache()
            dit = {}
            for name, dense_attn in (("token2tile", False), ("dense", True)):
                rec = dit_measure(rank, world, dev, dist.group.WORLD, dense_attention=dense_attn, steps=4, warmup=4,
                                  with_e2e=False)
                if rec is not None:
                    dit[name] = {"ms_per_step": rec["value"], "config": rec["config"], "clocks": rec["clocks"],
                                 "gemm_TFLOPs": rec["roofline"]["achieved"], "gpu_launches": rec["gpu_launches"]}
            if rank == 0 and "dense" in dit and "token2tile" in dit:
                dit["speedup_vs_dense_attention"] = dit["dense"]["ms_per_step"] / dit["token2tile"]["ms_per_step"]
        except Exception as exc:      # noqa: BLE001 - the headline metric does not depend on it
            print(f"[bench] transformer step skipped: {type(exc).__name__}: {exc}", file=sys.stderr)
            dit = None

    pk = peaks()
    flops = 4.0 * W["D"] * pairs
    t_attn = stages.get("attn_exact", 0.0)
    roofline = None
    if t_attn > 0:
        ach = flops / (t_attn * 1e-3) / 1e12
        # DRAM bytes of the two attention kernels: dram__bytes_read + dram__bytes_write of one ncu capture of the
        # 8-head 480p case, scaled by the rows processed (each kernel reads q, kp, vp once; the exact output is
        # written once: traffic is proportional to H * N)
        traffic = ATTN_DRAM_BYTES_480P_8H * (Hl * float(N)) / (8 * 32760.0)
        roofline = {"kernel": "attn2_kernel + attn_kernel (exact tile attention)", "bound": "tensor", "achieved": ach, "peak": pk["tf"],
                    "unit": "TFLOP/s", "frac": ach / pk["tf"], "traffic": traffic,
                    "traffic_source": "ncu 480p x 8 heads capture scaled by rows", "peak_source": pk["src"] +
                    " (sustained bf16 GEMM)", "flops_per_launch": flops, "ms_per_launch": t_attn,
                    "executed_pair_fraction": pairs / (Hl * float(N) * N)}
    B = 2
    stage_bytes = {
        "project": 2 * N * W["D"] * B * Hl + 2 * N * 32 * B * Hl,
        "gather_k": 2 * N * W["D"] * B * Hl,
        "kmeans": (6 * N * 32 * B + 2 * N * W["D"] * B + 10 * N * 4) * Hl,
        "vstats": 2 * N * W["D"] * B * Hl,
    }
    # gather_k and vstats are timed in the reuse call, where they run alone on the main stream (in a rebuild
    # call the key gather runs on the side stream under the selection and the value statistics are part of
    # the clustering stage)
    stage_ms = dict(stages)
    for n in ("gather_k", "vstats"):
        if reuse_stages.get(n):
            stage_ms[n] = reuse_stages[n]
    stage_roof = {}
    for n in stage_bytes:
        if stage_ms.get(n):
            gbs = stage_bytes[n] / (stage_ms[n] * 1e-3) / 1e9
            if gbs <= 1.05 * pk["hbm"]:          # anything above the copy peak is a timing artefact, not a result
                stage_roof[n] = {"ms": stage_ms[n], "algorithmic_GBps": gbs, "frac_of_hbm_peak": gbs / pk["hbm"],
                                 "timed_in": "reuse call" if n in ("gather_k", "vstats") else "rebuild call"}
    if stages.get("select"):
        # scoring + selection: N * C scores per head; bound by integer / compare issue, so both nominal
        # fractions are reported next to the score rate
        t_sel = stages["select"] * 1e-3
        scores = float(N) * 2048 * Hl
        sel_bytes = (N * 32 * B + 2048 * 32 * B + CQ * 2048 / 8) * Hl
        stage_roof["select"] = {"ms": stages["select"], "scores_per_s": scores / t_sel,
                                "TFLOPs": 2 * 32 * scores / t_sel / 1e12,
                                "frac_of_tensor_peak": 2 * 32 * scores / t_sel / 1e12 / pk["tf"],
                                "algorithmic_GBps": sel_bytes / t_sel / 1e9,
                                "frac_of_hbm_peak": sel_bytes / t_sel / 1e9 / pk["hbm"],
                                "bound": "integer / compare instruction issue (about 22 instructions per score over the two passes)"}
    tail_flops = float(N) * 2048 * (2 * 32 + 2 * W["D"]) * Hl
    if stages.get("residual_merge"):
        stage_roof["residual_merge"] = {"ms": stages["residual_merge"],
                                        "TFLOPs": tail_flops / (stages["residual_merge"] * 1e-3) / 1e12,
                                        "frac_of_tensor_peak": tail_flops / (stages["residual_merge"] * 1e-3) / 1e12 / pk["tf"]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        step, cores = cpu_head_step_factory()
        val = step()
        cpu = {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": "one head of 40 (full 75,600 tokens), one rebuild call, time x 40 (an extrapolation; "
                         "cpu_config below is measured whole)"}
        try:      # the CPU-sized configuration as a whole: H 2, N 4096, CQ 32, fp32, 5 % budget
            cpu["cpu_config"] = cpu_small_config()
        except Exception as exc:      # noqa: BLE001 - informative only
            print(f"[bench] CPU configuration skipped: {type(exc).__name__}: {exc}", file=sys.stderr)

    if rank == 0:
        amort = (ms_step + 7 * reuse_ms) / 8
        bytes_in = 3 * Hl * N * W["D"] * 2
        line = {
            "metric": METRIC, "value": ms_step, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": W["name"], "H": W["H"], "heads_per_gpu": Hl, "N": N, "CQ": CQ, "D": W["D"],
                       "budget": W["s_frac"], "ns": ns_layer, "call": "rebuild (mask_refresh=1)",
                       "parallelism": f"head-parallel x{world}", "l2": "inputs (2.3 GB/step) exceed L2; no flush"},
            "roofline": roofline, "cpu_baseline": cpu,
            "e2e": {"value": e2e_ms, "unit": UNIT, "h2d_bytes_per_step": bytes_in,
                    "d2h_bytes_per_step": Hl * N * W["D"] * 2,
                    "h2d_GBps_this_rank": bytes_in / (e2e_ms * 1e-3) / 1e9,
                    "mode": "double-buffered inputs and outputs: the copies of a step overlap the neighbouring steps' compute",
                    "serial_ms": e2e_serial_ms},
            "gpu_launches": KERNELS_REBUILD * args.steps, "clocks": clocks,
            "reuse_ms": reuse_ms, "amortised_ms_1_rebuild_7_reuse": amort, "stages_ms": stages,
            "reuse_stages_ms": reuse_stages, "stage_roofline": stage_roof, "tasks": tasks, "m_utilisation": m_util,
            "dense_ms": dense, "fastest_dense_ms": dense_best, "budgets": budgets, "init_ms": init_ms,
            "config_480p": config2, "dit_step_ulysses8": dit,
            "speedup_vs_dense": {"rebuild": dense_best / ms_step, "reuse": dense_best / reuse_ms,
                                 "amortised": dense_best / amort} if dense_best else None,
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------
# full transformer step (40 blocks, Ulysses sequence parallelism at N > 1)
# ---------------------------------------------------------------------------

def dit_measure(rank, world, dev, group, *, grid_name="720p", blocks=0, dense_attention=False, steps=4, warmup=4,
                with_e2e=True):
    """One denoising step = both CFG branches through all blocks.  The timed steps cover whole refresh periods
    of the structure (mask_refresh = 4): the first step of a period rebuilds in branch 0, everything else
    reuses.  Returns the bench record of the workload (rank 0) or None; the process group, if any, is the
    caller's."""
    import torch.distributed as dist
    from token2tile_b200 import dit_step as D
    from token2tile_b200 import t2t_attn as B
    from token2tile_b200.synth import GRIDS

    B.clear_runtimes()
    B.set_ulysses_world_size(world)
    shape = D.WAN_14B
    grid = GRIDS[grid_name]
    N = grid[0] * grid[1] * grid[2]
    CQ = {75600: 512, 32760: 256}.get(N, max(32, N // 128))
    ns = max(1, int(0.015 * N))
    if N % world or shape.heads % world:
        raise SystemExit(f"{N} tokens / {shape.heads} heads do not split over {world} ranks")
    B.set_backend_config({"t2t_fast_init": True})

    class DenseImpl:
        def __init__(self, num_heads, head_size, causal, softmax_scale, prefix=""):
            self.dense = B.DenseAttention(num_heads, head_size, softmax_scale)

        def forward(self, q, k, v, meta):
            return self.dense.forward(q, k, v)

    nblocks = blocks or shape.blocks
    model = D.DiTStep(shape, device=dev, seed=0, group=group, blocks=nblocks,
                      make_attn=DenseImpl if dense_attention else None)
    # residual stream: a locality mixture in the model width (512 centres, blocks of 1x4x4 tokens)
    g = torch.Generator(device=dev).manual_seed(1234)
    T, Y, X = grid
    t = torch.arange(T, device=dev)[:, None, None].expand(T, Y, X)
    y = torch.arange(Y, device=dev)[None, :, None].expand(T, Y, X)
    x = torch.arange(X, device=dev)[None, None, :].expand(T, Y, X)
    by, bx = (Y + 3) // 4, (X + 3) // 4
    block = ((t * by + y // 4) * bx + x // 4).reshape(N)
    cen = torch.randn(512, shape.dim, generator=g, device=dev)
    pick = torch.randint(0, 512, (T * by * bx,), generator=g, device=dev)
    n = N // world
    rows = slice(rank * n, (rank + 1) * n)
    noise = torch.randn(N, shape.dim, generator=g, device=dev)[rows]
    x_dev = (cen[pick[block[rows]]] + 0.3 * noise).to(torch.bfloat16).contiguous()
    del noise
    text = torch.randn(shape.text_len, shape.text_dim, generator=g, device=dev).to(torch.bfloat16)
    hx = x_dev.cpu().pin_memory()
    hout = torch.empty_like(hx).pin_memory()

    build = B.T2TAttentionMetadataBuilder().build
    cache = B.T2TRequestCache()

    def meta(step):
        return build(step, 50, cache, profile_name="manual", ns_base=ns, dense_prefix_steps=0, cq=CQ, ck=2048,
                     step_profile=(1.0,) * 4, layer_profile=(1.0,) * 6, cfg_mult=(1.0, 1.0), mask_refresh=4,
                     cfg_reuse=True)

    counter = [0]

    def denoise_step(host=False):
        step = counter[0]
        counter[0] += 1
        m = meta(step)
        if host:
            x_dev.copy_(hx, non_blocking=True)
        for branch in range(2):
            out = model.forward(x_dev, text, 999.0 - 20 * step, m)
        if host:
            hout.copy_(out, non_blocking=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def maxr(v):
        if world == 1:
            return v
        tt = torch.tensor([v], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    warm = max(4, (warmup + 3) // 4 * 4)       # whole refresh periods, so the timed steps start with a rebuild
    for _ in range(warm):
        denoise_step()
    barrier()
    sampler = ClockSampler(dev.index or 0) if rank == 0 else None
    rebuilds = sum(1 for s_ in range(counter[0], counter[0] + steps) if s_ % 4 == 0)   # branch-0 calls that rebuild
    ms = time_events(denoise_step, steps)
    barrier()
    clocks = sampler.stop() if sampler else None
    ms_step = maxr(ms / steps)
    e2e_ms = None
    if with_e2e:
        counter[0] = (counter[0] + 3) // 4 * 4
        denoise_step(host=True)
        barrier()
        counter[0] = (counter[0] + 3) // 4 * 4
        e2e_ms = maxr(time_events(lambda: denoise_step(host=True), steps) / steps)
        barrier()
    if not dense_attention:
        for rt in B._RUNTIMES.values():
            assert rt.deploy.device_status() == 0, "a device wait timed out"
    line = None
    if rank == 0:
        pk = peaks()
        gemm_flops = 2 * D.flops_per_step(D.DiTShape(blocks=nblocks), N) / world      # two branches, this rank's tokens
        line = {
            "metric": "dit_denoising_step_ms", "value": ms_step, "unit": "ms/step", "n_gpus": world, "steps": steps,
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "wan2.1-14b-shaped-dit-step-" + grid_name, "blocks": nblocks,
                       "dim": shape.dim, "heads": shape.heads, "ffn": shape.ffn, "N": N, "text_tokens": shape.text_len,
                       "cfg_branches_per_step": 2, "rebuild_steps_in_timed_region": rebuilds, "self_attention": "dense" if dense_attention else
                       f"token2tile ns={ns} CQ={CQ} mask_refresh=4 cfg_reuse", "parallelism": f"ulysses x{world}",
                       "weights_GB": model.weight_bytes() / 1e9,
                       "all_to_all_bytes_per_rank_per_block": D.all_to_all_bytes_per_block(shape, N, world),
                       "l2": "activations (0.77 GB per tensor) exceed L2; no flush"},
            "roofline": {"kernel": "dense GEMMs of the step (cuBLAS)", "bound": "tensor",
                         "achieved": gemm_flops / (ms_step * 1e-3) / 1e12, "peak": pk["tf"], "unit": "TFLOP/s",
                         "frac": gemm_flops / (ms_step * 1e-3) / 1e12 / pk["tf"], "traffic": None,
                         "note": "GEMM FLOPs only over the whole step time: a lower bound on utilisation"},
            "cpu_baseline": None,
            "e2e": {"value": e2e_ms, "unit": "ms/step", "h2d_bytes_per_step": hx.numel() * 2,
                    "d2h_bytes_per_step": hout.numel() * 2} if with_e2e else None,
            "gpu_launches": None if dense_attention else
            nblocks * (rebuilds * KERNELS_REBUILD + (2 * steps - rebuilds) * KERNELS_REUSE),
            "clocks": clocks,
        }
    del model, x_dev, hx, hout
    B.clear_runtimes()
    torch.cuda.empty_cache()
    return line


def run_dit(args, rank, world, local_rank):
    import torch.distributed as dist
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    group = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    line = dit_measure(rank, world, dev, group, grid_name=args.grid or "720p", blocks=args.blocks,
                       dense_attention=args.dense_attention, steps=args.steps, warmup=args.warmup)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--heads", type=int, default=0, help="override the head count (profiling cases)")
    ap.add_argument("--grid", default="", choices=["", "cpu", "480p", "720p"], help="override the latent grid")
    ap.add_argument("--light", action="store_true", help="timed steps and stage times only")
    ap.add_argument("--workload", default="layer", choices=["layer", "dit_step"],
                    help="layer: one attention layer (the headline metric); dit_step: a full transformer step")
    ap.add_argument("--blocks", type=int, default=0, help="dit_step: number of blocks (default 40)")
    ap.add_argument("--dense-attention", action="store_true", help="dit_step: dense self-attention instead")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
    else:
        if args.warmup < 3:
            args.warmup = 3
        if args.workload == "dit_step":
            run_dit(args, rank, world, local_rank)
        else:
            run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
