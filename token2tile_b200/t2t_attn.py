"""SGLang attention backend around the Token2Tile operator (B200 build).

Mirror of the reference's backend module
(integrations/sglang/backend/t2t_attn.py): the same classes, argument names
and request lifecycle, over `token2tile_b200.deploy_step.MaskedStepDeploy`.
The backend owns everything around the operator call:

  * the dense prefix: the first `dense_prefix_steps` denoising steps run plain
    dense attention (t2t_attn.py:1104-1107);
  * the budget schedule: a token budget per (step window, layer, CFG branch),
    written into the operator's device-side `ns_t` before every call
    (t2t_attn.py:561-589, 688-720, 1169-1177);
  * the per-request cache: projections and centroids per (layer, branch), CFG
    branch counting per (step, layer), snapshot reset when a new request starts
    (t2t_attn.py:332-339, 1138-1155, 1180-1192);
  * the packed [context | video] path of the second model family
    (`forward_varlen`, t2t_attn.py:1209-1412): context rows dense, context keys
    pinned as one always-selected key cluster, video rows through the operator.

Tensors are bfloat16 here (float16 in the reference).  When SGLang is
importable its base classes, dense FlashAttention implementation, forward
context and server arguments are used; otherwise small local stand-ins with
the same surface keep the module usable and testable on its own.
"""
from __future__ import annotations

import enum
import hashlib
import json
import math
import re
import threading
from dataclasses import dataclass, field
from pathlib import Path
from types import SimpleNamespace
from typing import Any

import torch

KERNEL_DTYPE = torch.bfloat16

# ---------------------------------------------------------------------------
# host framework: SGLang when present, local stand-ins otherwise
# ---------------------------------------------------------------------------
try:  # pragma: no cover - SGLang is an optional host
    from sglang.multimodal_gen.runtime.layers.attention.backends.attention_backend import (
        AttentionBackend,
        AttentionImpl,
        AttentionMetadata,
        AttentionMetadataBuilder,
    )
    from sglang.multimodal_gen.runtime.layers.attention.backends.flash_attn import (
        FlashAttentionImpl as _HostDenseImpl,
        FlashAttentionMetadata as _HostDenseMetadata,
    )
    from sglang.multimodal_gen.runtime.distributed.parallel_state import (
        get_ulysses_parallel_world_size as _host_ulysses_world_size,
    )
    from sglang.multimodal_gen.runtime.managers.forward_context import (
        get_forward_context as _host_forward_context,
    )
    from sglang.multimodal_gen.runtime.platforms import AttentionBackendEnum
    from sglang.multimodal_gen.runtime.server_args import (
        get_global_server_args as _host_server_args,
    )
    HAVE_SGLANG = True
except ImportError:
    HAVE_SGLANG = False

    class AttentionBackend:
        """Stand-in for SGLang's backend descriptor class."""
        accept_output_buffer: bool = False

    class AttentionImpl:
        """Stand-in for SGLang's per-layer attention implementation class."""

    @dataclass
    class AttentionMetadata:
        current_timestep: int

    class AttentionMetadataBuilder:
        """Stand-in for SGLang's metadata builder class."""

    class AttentionBackendEnum(enum.Enum):
        FA = "fa"
        T2T_ATTN = "t2t_attn"

    _HostDenseImpl = None
    _HostDenseMetadata = None
    _host_ulysses_world_size = None
    _host_forward_context = None
    _host_server_args = None


# What the stand-ins read when SGLang is absent: tests and stand-alone hosts
# set these through the three setters below.
_LOCAL = SimpleNamespace(backend_config={}, forward_context=None, ulysses=1)


def set_backend_config(config: dict[str, Any] | None) -> None:
    """Stand-alone replacement for the server's `attention_backend_config`."""
    _LOCAL.backend_config = dict(config or {})


def set_forward_context(context: Any) -> None:
    """Stand-alone replacement for SGLang's forward context: any object with
    `current_timestep` and, for the packed path, `minimax_h3_layout`."""
    _LOCAL.forward_context = context


def set_ulysses_world_size(n: int) -> None:
    """Stand-alone replacement for the sequence-parallel group size."""
    _LOCAL.ulysses = max(1, int(n))


def _backend_config() -> dict[str, Any]:
    if _host_server_args is not None:
        try:
            return getattr(_host_server_args(), "attention_backend_config", None) or {}
        except Exception:  # noqa: BLE001 - server arguments not initialised
            return {}
    return _LOCAL.backend_config


def _forward_context():
    if _host_forward_context is not None:
        try:
            return _host_forward_context()
        except AssertionError:
            return None
    return _LOCAL.forward_context


def _ulysses_world_size() -> int:
    """Head-sharding degree of this rank's sequence-parallel group; 1 when no
    group exists (t2t_attn.py:54-60)."""
    if _host_ulysses_world_size is not None:
        try:
            return max(1, int(_host_ulysses_world_size()))
        except Exception:  # noqa: BLE001 - distributed state not initialised
            return 1
    return _LOCAL.ulysses


class DenseAttention:
    """Dense attention of the prefix steps and of the context rows.  SGLang's
    FlashAttention implementation when hosted; torch's fused scaled-dot-product
    attention otherwise.  Tensors: [B, N, H, D] (`forward`) or packed
    [T, H, D] (`forward_varlen`, one document of `max_seqlen` rows)."""

    def __init__(self, num_heads, head_size, softmax_scale, num_kv_heads=None, prefix=""):
        self.scale = softmax_scale
        self._host = None
        if _HostDenseImpl is not None:
            self._host = _HostDenseImpl(num_heads=num_heads, head_size=head_size, causal=False,
                                        softmax_scale=softmax_scale, num_kv_heads=num_kv_heads, prefix=prefix)

    def forward(self, query, key, value):
        if self._host is not None:
            return self._host.forward(query, key, value, _HostDenseMetadata())
        out = torch.nn.functional.scaled_dot_product_attention(
            query.transpose(1, 2), key.transpose(1, 2), value.transpose(1, 2), scale=self.scale)
        return out.transpose(1, 2).contiguous()

    def forward_varlen(self, query, key, value, *, cu_seqlens, max_seqlen, cu_seqlens_host=None):
        if self._host is not None:
            return self._host.forward_varlen(query, key, value, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen,
                                             cu_seqlens_host=cu_seqlens_host)
        bounds = cu_seqlens_host if cu_seqlens_host is not None else tuple(int(x) for x in cu_seqlens.tolist())
        out = torch.zeros_like(query)
        for a, b in zip(bounds[:-1], bounds[1:]):
            if b > a:
                out[a:b] = self.rows_over(query[a:b], key[a:b], value[a:b])
        return out

    def rows_over(self, q_rows, keys, values):
        """Attention of q_rows [R, H, D] over keys / values [T, H, D]."""
        out = torch.nn.functional.scaled_dot_product_attention(
            q_rows.transpose(0, 1), keys.transpose(0, 1), values.transpose(0, 1), scale=self.scale)
        return out.transpose(0, 1)


# ---------------------------------------------------------------------------
# budget schedule
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class T2TProfile:
    """Budget profile of one workload geometry (t2t_attn.py:69-83): the base
    token budget, the number of dense prefix steps, the cluster counts and the
    multipliers per step window, per layer (6 groups or one per layer) and per
    CFG branch."""

    name: str
    num_heads: int
    seq_len: int
    total_steps: int
    ns_base: int
    dense_prefix_steps: int
    cq: int
    ck: int
    step_profile: tuple[float, ...]
    layer_profile: tuple[float, ...]
    cfg_mult: tuple[float, float] = (1.0, 1.0)


# Frozen multipliers of the built-in profiles (t2t_attn.py:86-94).
DEFAULT_STEP_PROFILE = (1.574482, 0.985902, 0.555188, 0.884428)
DEFAULT_LAYER_PROFILE = (1.189098, 1.123097, 1.278643, 0.915148, 0.956427, 0.537588)


def _builtin(name, heads, seq_len, ns_base, cq):
    return T2TProfile(name=name, num_heads=heads, seq_len=seq_len, total_steps=50, ns_base=ns_base,
                      dense_prefix_steps=12, cq=cq, ck=2048, step_profile=DEFAULT_STEP_PROFILE,
                      layer_profile=DEFAULT_LAYER_PROFILE)


# Profiles selected by profile_name="auto" on an exact (heads, tokens, steps)
# match (t2t_attn.py:96-136).
BUILTIN_PROFILES = {
    p.name: p for p in (
        _builtin("wan21_t2v_n32760_t50", 12, 32760, 1050, 256),
        _builtin("wan21_t2v_1_3b_n75600_t50", 12, 75600, 2424, 512),
        _builtin("wan21_t2v_14b_n75600_t50", 40, 75600, 2424, 512),
    )
}

# layers of the models the profiles are defined for, by head count (t2t_attn.py:455-464)
_LAYERS_BY_HEADS = {12: 30, 40: 40, 56: 50}


def profile_num_layers(profile: T2TProfile) -> int:
    try:
        return _LAYERS_BY_HEADS[profile.num_heads]
    except KeyError:
        raise ValueError(f"Unsupported head count H={profile.num_heads}: layer counts are known for "
                         "12, 40 and 56 heads") from None


def validate_profile(profile: T2TProfile) -> None:
    """Shape and range checks of a profile (t2t_attn.py:467-479)."""
    layers = profile_num_layers(profile)
    if len(profile.step_profile) != 4 or len(profile.layer_profile) not in (6, layers):
        raise ValueError(f"Invalid Token2Tile profile shape: {profile.name}")
    if len(profile.cfg_mult) != 2:
        raise ValueError(f"Invalid Token2Tile CFG profile shape: {profile.name}")
    if not 0 < profile.ns_base <= profile.seq_len:
        raise ValueError(f"Invalid Token2Tile ns_base: {profile.name}")
    if profile.dense_prefix_steps < 0 or profile.cq <= 0 or profile.ck <= 0:
        raise ValueError(f"Invalid Token2Tile profile constants: {profile.name}")


_MANUAL_KEYS = ("ns_base", "dense_prefix_steps", "cq", "ck", "step_profile", "layer_profile", "cfg_mult")


def resolve_profile(metadata, seq_len: int, num_heads: int) -> T2TProfile:
    """Profile of a call (t2t_attn.py:482-558).  "manual" needs every budget
    key; a built-in profile accepts none of them and must match the geometry
    exactly; "auto" picks the one built-in profile that matches."""
    manual = {k: getattr(metadata, k) for k in _MANUAL_KEYS}
    supported = ", ".join(sorted(BUILTIN_PROFILES))
    if metadata.profile_name == "manual":
        if any(v is None for v in manual.values()):
            raise ValueError("t2t_profile='manual' requires ns_base, dense_prefix_steps, cq, ck, step_profile, "
                             "layer_profile, and cfg_mult")
        profile = T2TProfile(name="manual", num_heads=num_heads, seq_len=seq_len, total_steps=metadata.total_steps,
                             ns_base=int(manual["ns_base"]), dense_prefix_steps=int(manual["dense_prefix_steps"]),
                             cq=int(manual["cq"]), ck=int(manual["ck"]), step_profile=tuple(manual["step_profile"]),
                             layer_profile=tuple(manual["layer_profile"]), cfg_mult=tuple(manual["cfg_mult"]))
    else:
        if any(v is not None for v in manual.values()):
            raise ValueError("Token2Tile budget keys require t2t_profile='manual'; built-in profiles cannot be "
                             "partially overridden")
        geometry = (num_heads, seq_len, metadata.total_steps)
        if metadata.profile_name == "auto":
            hits = [p for p in BUILTIN_PROFILES.values() if (p.num_heads, p.seq_len, p.total_steps) == geometry]
            if len(hits) != 1:
                raise ValueError(f"No built-in Token2Tile profile for H={num_heads}, N={seq_len}, "
                                 f"steps={metadata.total_steps}. Supported: {supported}")
            profile = hits[0]
        else:
            profile = BUILTIN_PROFILES.get(metadata.profile_name)
            if profile is None:
                raise ValueError(f"Unknown Token2Tile profile {metadata.profile_name!r}. "
                                 f"Supported: auto, manual, {supported}")
            if (profile.num_heads, profile.seq_len, profile.total_steps) != geometry:
                raise ValueError(f"Token2Tile profile {profile.name} expects H={profile.num_heads}, "
                                 f"N={profile.seq_len}, steps={profile.total_steps}; got H={num_heads}, "
                                 f"N={seq_len}, steps={metadata.total_steps}")
    validate_profile(profile)
    return profile


def step_window(step: int) -> int:
    """Step window of a denoising step of a 50-step schedule: boundaries at
    steps 21, 31 and 41 (t2t_attn.py:561-570).  The budget is only read by
    rebuild calls."""
    return (step >= 21) + (step >= 31) + (step >= 41)


def layer_factor(layer_idx: int, profile: T2TProfile) -> float:
    """Layer multiplier: one per layer, or six groups of nearly equal size
    (t2t_attn.py:573-589)."""
    layers = profile_num_layers(profile)
    if not 0 <= layer_idx < layers:
        raise ValueError(f"Token2Tile layer index {layer_idx} is outside [0, {layers})")
    if len(profile.layer_profile) == layers:
        return profile.layer_profile[layer_idx]
    return profile.layer_profile[min(layer_idx * 6 // layers, 5)]


def budget(ns_base: int, step_mult: float, layer_mult: float, cfg_mult: float, seq_len: int) -> int:
    """round(ns_base * multipliers) clamped to [1, seq_len] (t2t_attn.py:689-702)."""
    return min(seq_len, max(1, int(round(ns_base * step_mult * layer_mult * cfg_mult))))


def budget_map(profile: T2TProfile, seq_len: int, table_rows=None) -> dict[tuple[int, int, int], int]:
    """Token budget per (window, layer, CFG branch) (t2t_attn.py:687-716).  An
    exact table replaces the product for both branches; cfg_mult is not applied
    on top of a table."""
    layers = profile_num_layers(profile)
    out = {}
    for w in range(4):
        for layer in range(layers):
            for cfg in range(2):
                if table_rows is not None:
                    out[(w, layer, cfg)] = table_rows[w][layer]
                else:
                    out[(w, layer, cfg)] = budget(profile.ns_base, profile.step_profile[w],
                                                  layer_factor(layer, profile), profile.cfg_mult[cfg], seq_len)
    return out


def load_ns_table(path: str, *, expected_layers: int, max_ns: int):
    """Exact per-(window, layer) budgets from a JSON file of schema
    "t2t_ns_table_v1": {"schema", "heads", "seq_len", "ns": 4 rows of
    expected_layers ints in (0, max_ns]} (t2t_attn.py:592-616).  Returns
    (rows, sha256 of the file, the parsed header); geometry checks are the
    caller's."""
    table_path = Path(path).resolve()
    raw = table_path.read_bytes()
    data = json.loads(raw)
    if data.get("schema") != "t2t_ns_table_v1":
        raise ValueError(f"Unsupported Token2Tile ns-table schema in {table_path}")
    rows = tuple(tuple(int(v) for v in row) for row in data["ns"])
    if len(rows) != 4 or any(len(row) != expected_layers for row in rows):
        raise ValueError(f"Token2Tile ns-table {table_path} must be 4x{expected_layers}")
    if any(not 0 < v <= max_ns for row in rows for v in row):
        raise ValueError(f"Token2Tile ns-table {table_path} has ns outside (0, {max_ns}]")
    return rows, hashlib.sha256(raw).hexdigest(), data


# ---------------------------------------------------------------------------
# request cache, metadata, backend descriptor
# ---------------------------------------------------------------------------
@dataclass
class T2TRequestCache:
    """State of one generation request (t2t_attn.py:332-339): operator state
    per (layer, CFG branch), calls seen per (step, layer), and the runtime the
    request is bound to."""
    states: dict[tuple[int, int], dict[str, torch.Tensor]] = field(default_factory=dict)
    call_counts: dict[tuple[int, int], int] = field(default_factory=dict)
    runtime_key: tuple[Any, ...] | None = None
    initialized_runtime: bool = False


@dataclass
class T2TAttentionMetadata(AttentionMetadata):
    """Per-step metadata handed to every layer (t2t_attn.py:342-363)."""
    step_index: int
    total_steps: int
    profile_name: str
    ns_base: int | None
    dense_prefix_steps: int | None
    cq: int | None
    ck: int | None
    step_profile: tuple[float, ...] | None
    layer_profile: tuple[float, ...] | None
    cfg_mult: tuple[float, ...] | None
    ns_table: str | None
    warm_iters: int
    mask_refresh: int
    cfg_reuse: bool
    use_kmm: bool          # accepted for compatibility; has no effect
    cache: T2TRequestCache
    # dense cross-attention reads the same metadata object and uses these two
    max_seqlen_q: int | None = None
    max_seqlen_k: int | None = None


def _opt(convert, value):
    return None if value is None else convert(value)


def _floats(values):
    return tuple(float(v) for v in values)


class T2TAttentionMetadataBuilder(AttentionMetadataBuilder):
    def __init__(self) -> None:
        pass

    def prepare(self) -> None:
        pass

    def build(self, step_index: int, total_steps: int, cache: T2TRequestCache, profile_name: str = "auto",
              ns_base=None, dense_prefix_steps=None, cq=None, ck=None, step_profile=None, layer_profile=None,
              cfg_mult=None, ns_table=None, warm_iters: int = 4, mask_refresh: int = 4, cfg_reuse: bool = True,
              use_kmm: bool = True, **kwargs: Any) -> T2TAttentionMetadata:
        """Normalises the pipeline's arguments (t2t_attn.py:373-417); unknown
        keyword arguments are ignored as in the reference."""
        return T2TAttentionMetadata(
            current_timestep=int(step_index), step_index=int(step_index), total_steps=int(total_steps),
            profile_name=str(profile_name), ns_base=_opt(int, ns_base),
            dense_prefix_steps=_opt(int, dense_prefix_steps), cq=_opt(int, cq), ck=_opt(int, ck),
            step_profile=_opt(_floats, step_profile), layer_profile=_opt(_floats, layer_profile),
            cfg_mult=_opt(_floats, cfg_mult), ns_table=_opt(str, ns_table), warm_iters=int(warm_iters),
            mask_refresh=int(mask_refresh), cfg_reuse=bool(cfg_reuse), use_kmm=bool(use_kmm), cache=cache)


class T2TAttentionBackend(AttentionBackend):
    """Backend descriptor (t2t_attn.py:420-441)."""
    accept_output_buffer: bool = True

    @staticmethod
    def get_supported_head_sizes() -> list[int]:
        return [128]

    @staticmethod
    def get_enum():
        return AttentionBackendEnum.T2T_ATTN

    @staticmethod
    def get_impl_cls():
        return T2TAttentionImpl

    @staticmethod
    def get_metadata_cls():
        return T2TAttentionMetadata

    @staticmethod
    def get_builder_cls():
        return T2TAttentionMetadataBuilder


def device_supported(device=None) -> bool:
    """The kernels are sm_100a only: compute capability (10, 0).  The reference's
    registration gates on (9, 0) at the same place (token2tile_sglang.patch:103-109)."""
    return torch.cuda.is_available() and torch.cuda.get_device_capability(device) == (10, 0)


# ---------------------------------------------------------------------------
# operator module and runtimes
# ---------------------------------------------------------------------------
_MODULE_LOCK = threading.Lock()
_OPERATOR_MODULES: dict[str, Any] = {}
_RUNTIME_LOCK = threading.Lock()
_RUNTIMES: dict[tuple[Any, ...], "_T2TRuntime"] = {}
_H3_RUNTIMES: dict[tuple[Any, ...], "_H3Runtime"] = {}


def _load_operator(tag: str):
    """Operator module of a model path, "wan" or "h3" (t2t_attn.py:308-329).
    One module object serves both here: the per-path differences of the
    reference (which projection fit runs) are instance-level in this build."""
    with _MODULE_LOCK:
        module = _OPERATOR_MODULES.get(tag)
        if module is None:
            from . import deploy_step as module
            _OPERATOR_MODULES[tag] = module
        return module


def clear_runtimes() -> None:
    """Drop every cached operator instance (frees their device buffers)."""
    with _RUNTIME_LOCK:
        _RUNTIMES.clear()
        _H3_RUNTIMES.clear()


@dataclass
class _T2TRuntime:
    """One operator instance and its budget schedule; shared by every layer and
    request of the same geometry and settings (t2t_attn.py:444-452)."""
    module: Any
    deploy: Any
    key: tuple[Any, ...]
    profile: T2TProfile
    ns_map: dict[tuple[int, int, int], int]
    ns_tensors: dict[int, torch.Tensor]
    active_cache_id: int | None = None


def _ns_tensors(values, deploy, device):
    """One 0-dim device tensor per distinct budget, so that setting the budget
    is a device-to-device copy on the operator's stream (no host sync)."""
    return {v: torch.tensor(v, device=device, dtype=deploy.ns_t.dtype) for v in set(values)}


def _get_runtime(metadata, profile, heads, seq_len, head_dim, device, total_heads=None) -> _T2TRuntime:
    """Runtime for this geometry and these settings (t2t_attn.py:619-748).
    `heads` is the local head count of this rank; the budget table's geometry
    is checked against the model's total head count."""
    total_heads = heads if total_heads is None else int(total_heads)
    table = None
    if metadata.ns_table is not None:
        rows, digest, header = load_ns_table(metadata.ns_table, expected_layers=profile_num_layers(profile),
                                             max_ns=seq_len)
        if int(header["heads"]) != total_heads or int(header["seq_len"]) != seq_len:
            raise ValueError(f"Token2Tile ns-table geometry mismatch: table H={header['heads']} "
                             f"N={header['seq_len']} vs runtime H={total_heads} (local {heads}) N={seq_len}")
        table = (rows, digest)
    key = (heads, total_heads, seq_len, head_dim, profile, metadata.mask_refresh, metadata.cfg_reuse,
           metadata.use_kmm, str(device), metadata.ns_table, None if table is None else table[1])
    with _RUNTIME_LOCK:
        runtime = _RUNTIMES.get(key)
        if runtime is not None:
            return runtime
        module = _load_operator("wan")
        deploy = module.MaskedStepDeploy(heads, seq_len, profile.cq, C=profile.ck, D=head_dim,
                                         s_frac=profile.ns_base / seq_len, mask_refresh=metadata.mask_refresh,
                                         cfg_reuse=metadata.cfg_reuse, device=device)
        if bool(_backend_config().get("t2t_fast_init", False)):
            deploy.init_state = make_fast_init_state(deploy, module)
        ns_map = budget_map(profile, seq_len, None if table is None else table[0])
        runtime = _T2TRuntime(module=module, deploy=deploy, key=key, profile=profile, ns_map=ns_map,
                              ns_tensors=_ns_tensors(ns_map.values(), deploy, device))
        _RUNTIMES[key] = runtime
        return runtime


def _sanitize_state(state, previous) -> None:
    """Keep the previous centroid wherever the new one is non-finite or all
    zero (t2t_attn.py:751-760)."""
    for name in ("ck", "cq"):
        new, old = state[name], previous[name]
        newf = new.float()
        bad = (~torch.isfinite(newf).all(-1)) | (newf.abs().amax(-1) == 0)
        state[name] = torch.where(bad[..., None], old, new).contiguous()


def _order_after_caller(deploy, device) -> None:
    """The operator's streams wait for everything queued on the caller's
    stream (t2t_attn.py:1165-1167)."""
    if device.type == "cuda":
        current = torch.cuda.current_stream(device)
        deploy.s_main.wait_stream(current)
        deploy.s_side.wait_stream(current)


def _check_operator_status(deploy) -> None:
    """Waits for and examines the operator's device status word (an operator without the
    method - a stand-in, the reference's own class - is left alone)."""
    check = getattr(deploy, "check_status", None)
    if check is not None:
        check(wait=True)


def _set_budget(deploy, ns_tensor, device) -> None:
    """ns_t <- budget, ordered on the operator's main stream (t2t_attn.py:1176-1177)."""
    if device.type == "cuda":
        with torch.cuda.stream(deploy.s_main):
            deploy.ns_t.copy_(ns_tensor)
    else:
        deploy.ns_t.copy_(ns_tensor)


# ---------------------------------------------------------------------------
# fast state initialisation
# ---------------------------------------------------------------------------
def fast_online_u(qf, kf, r: int = 32):
    """The projection fit without the host-synchronising finiteness check
    (the reference's `_fast_online_u`, t2t_attn.py:211-239, moves the long
    products to fp32 tensor-core GEMMs and keeps only the 128x128
    factorisations in fp64).  Here `online_u` already works that way: both
    names run the same kernels (tensor-core second moments, fp64 Jacobi
    factorisations, batched over heads); this one returns as soon as the
    kernels are queued."""
    from .deploy_step import lowrank_fit
    return lowrank_fit(qf, kf, r, check_finite=False)


def make_fast_init_state(deploy, module=None):
    """`t2t_fast_init`: an `init_state` for `deploy` that never touches the host
    (the role of the reference's replacement, t2t_attn.py:260-281): projection
    fit without the finiteness read-back, first centroids drawn by a generator
    on the device, no trailing synchronisation.  Everything after the draw is
    the operator's own `warm_start`, so the Lloyd rounds are the same kernels
    as in `MaskedStepDeploy.init_state`."""

    def init_state(q, k, *, warm_iters=4, seed=0):
        with torch.cuda.device(deploy.dev):
            Uq, Uk = fast_online_u(q, k, deploy.r)
            gen = torch.Generator(device=deploy.dev).manual_seed(seed)

            def draw(count):
                return torch.randperm(deploy.N, generator=gen, device=deploy.dev)[:count].sort().values

            rows_k = draw(deploy.C)
            rows_q = draw(deploy.CQ)
            return deploy.warm_start(q, k, Uq, Uk, rows_k, rows_q, warm_iters)

    return init_state


# ---------------------------------------------------------------------------
# packed [context | video] documents (second model family)
# ---------------------------------------------------------------------------
@dataclass
class _H3Runtime:
    """Operator instance for one packed length (t2t_attn.py:800-811).  The
    operator sees `used_tokens` rows: the video rows first, then the context
    rows, whose keys are pinned (`pin_tail`)."""
    deploy: Any
    heads: int
    ns_map: dict[tuple[int, int], int]
    ns_tensors: dict[int, torch.Tensor]
    used_tokens: int
    video_tokens: int
    context_tokens: int
    mask_refresh: int
    cfg_reuse: bool
    dense_prefix: int


def _h3_config() -> dict[str, Any]:
    """Settings of the packed path, read from the backend configuration with
    the reference's keys and defaults (t2t_attn.py:819-866)."""
    cfg = _backend_config()
    step_profile = _floats(cfg.get("t2t_step_profile", DEFAULT_STEP_PROFILE))
    layer_profile = _floats(cfg.get("t2t_layer_profile", DEFAULT_LAYER_PROFILE))
    if len(step_profile) != 4 or len(layer_profile) != 6:
        raise ValueError("H3 Token2Tile needs 4 step and 6 layer multipliers")
    return {
        "video_tokens": int(cfg.get("t2t_h3_video_tokens", 0)),
        "s_frac": float(cfg.get("t2t_h3_s_frac", 0.05)),
        "dense_prefix": int(cfg.get("t2t_dense_prefix_steps", 12)),
        "mask_refresh": max(1, int(cfg.get("t2t_mask_refresh", 1))),
        "cfg_reuse": bool(cfg.get("t2t_cfg_reuse", False)),
        "cq": cfg.get("t2t_cq", "auto"),
        "ck": int(cfg.get("t2t_ck", 2048)),
        "step_profile": step_profile,
        "layer_profile": layer_profile,
        "ns_table": cfg.get("t2t_ns_table"),
        "warm_iters": int(cfg.get("t2t_warm_iters", 4)),
        # keep projections and centroids of the previous request of the same
        # geometry as the warm start of the next one
        "persist_state": bool(cfg.get("t2t_persist_state", False)),
        # "pin": keyframe condition rows are exact context; "sparse": they join
        # the generated rows in clustering and selection
        "cond_mode": str(cfg.get("t2t_h3_cond_mode", "pin")),
        "fast_init": bool(cfg.get("t2t_fast_init", False)),
        "sync_first_sparse": bool(cfg.get("t2t_sync_first_sparse", False)),
        "sync_init": bool(cfg.get("t2t_sync_init", False)),
    }


def _h3_layout():
    context = _forward_context()
    return getattr(context, "minimax_h3_layout", None) if context is not None else None


def _h3_split(used_tokens: int, cond_mode: str, device):
    """Where the sparse video rows of a packed document of `used_tokens` rows lie,
    from the layout the model publishes on the forward context
    (t2t_attn.py:869-908).  Returns (video_tokens, rows): video_tokens = 0 when
    this call is not the main packed document (then it stays dense); rows =
    None when the video rows are simply the tail of the document, else a pair
    (video row ids, context row ids) - the "sparse" condition mode, where the
    video rows are [condition rows | generated tail] and everything else is
    context."""
    layout = _h3_layout()
    if not layout:
        return 0, None
    video = int(layout.get("video", 0))
    stop_ok = layout.get("video_stop") == used_tokens
    if cond_mode == "sparse" and "video_tail" in layout and stop_ok:
        tail = int(layout["video_tail"])
        cond = video - tail
        if cond > 0:
            first = int(layout["video_start"])
            ids = torch.arange(used_tokens)
            is_video = ((ids >= first) & (ids < first + cond)) | (ids >= used_tokens - tail)
            return video, (ids[is_video].to(device), ids[~is_video].to(device))
    if video <= 0 or not stop_ok:
        return 0, None
    tail = int(layout.get("video_tail", video))
    if tail <= 0:
        return 0, None
    # without condition rows the video segment has to be the contiguous tail of the document
    if tail == video and layout["video_start"] != used_tokens - video:
        return 0, None
    return tail, None


def h3_auto_cq(used_tokens: int) -> int:
    """Query cluster count of the packed path when not configured: about one
    per 128 rows, a multiple of 4, at least 64 (t2t_attn.py:927-931)."""
    return max(64, int(round(used_tokens / 128 / 4)) * 4)


def _get_h3_runtime(used_tokens: int, device, heads: int = 28, video_tokens=None) -> _H3Runtime:
    """Runtime of the packed path (t2t_attn.py:911-1046): `heads` per kernel
    chunk; only runtimes of the current packed length are kept."""
    cfg = _h3_config()
    video_tokens = cfg["video_tokens"] if video_tokens is None else int(video_tokens)
    if not 0 < video_tokens < used_tokens:
        raise ValueError(f"t2t_h3_video_tokens must be in (0, {used_tokens}), got {video_tokens}")
    context_tokens = used_tokens - video_tokens
    cq = h3_auto_cq(used_tokens) if cfg["cq"] in (None, "auto") else int(cfg["cq"])
    table = None
    if cfg["ns_table"] is not None:
        rows, digest, header = load_ns_table(cfg["ns_table"], expected_layers=50, max_ns=used_tokens)
        # the packed length varies by a few tokens per prompt, and a table may
        # record the chunk (28) or the total (56) head count
        if int(header["heads"]) not in (28, 56) or abs(int(header["seq_len"]) - used_tokens) > 64:
            raise ValueError(f"Token2Tile H3 ns-table geometry mismatch: table H={header['heads']} "
                             f"N={header['seq_len']} vs runtime H=56 (chunk {heads}) N={used_tokens}")
        table = (rows, digest)
    key = (heads, used_tokens, video_tokens, cfg["s_frac"], cfg["dense_prefix"], cfg["mask_refresh"],
           cfg["cfg_reuse"], cq, cfg["ck"], cfg["step_profile"], cfg["layer_profile"], str(device),
           cfg["ns_table"], None if table is None else table[1])
    with _RUNTIME_LOCK:
        stale = [k for k in _H3_RUNTIMES if k[1] != used_tokens]
        for k in stale:
            _H3_RUNTIMES.pop(k)
        if stale and torch.cuda.is_available():
            import gc
            gc.collect()
            torch.cuda.empty_cache()
        runtime = _H3_RUNTIMES.get(key)
        if runtime is not None:
            return runtime
        module = _load_operator("h3")
        deploy = module.MaskedStepDeploy(heads, used_tokens, cq, C=cfg["ck"], D=128, r=32, s_frac=cfg["s_frac"],
                                         mask_refresh=cfg["mask_refresh"], cfg_reuse=cfg["cfg_reuse"],
                                         pin_tail=context_tokens, device=device)
        if cfg["fast_init"]:
            deploy.init_state = make_fast_init_state(deploy, module)
        ns_base = int(cfg["s_frac"] * used_tokens)
        ns_map = {}
        for w in range(4):
            for layer in range(50):
                if table is not None:
                    ns_map[(w, layer)] = min(used_tokens, table[0][w][layer])
                else:
                    ns_map[(w, layer)] = budget(ns_base, cfg["step_profile"][w],
                                                cfg["layer_profile"][min(layer * 6 // 50, 5)], 1.0, used_tokens)
        runtime = _H3Runtime(deploy=deploy, heads=heads, ns_map=ns_map,
                             ns_tensors=_ns_tensors(ns_map.values(), deploy, device), used_tokens=used_tokens,
                             video_tokens=video_tokens, context_tokens=context_tokens,
                             mask_refresh=cfg["mask_refresh"], cfg_reuse=cfg["cfg_reuse"],
                             dense_prefix=cfg["dense_prefix"])
        _H3_RUNTIMES[key] = runtime
        return runtime


# ---------------------------------------------------------------------------
# the per-layer implementation
# ---------------------------------------------------------------------------
def _heads_major(x):
    """[N, H, D] tensor -> [H, N, D] in the kernels' dtype WITHOUT a copy where possible: the kernels read
    whole-row strided views in place (the reference transposes and copies q, k and v here,
    t2t_attn.py:1161-1163).  A tensor of another dtype, with non-contiguous rows or on the CPU stand-in
    path is converted to a contiguous [H, N, D] copy as before."""
    view = x.transpose(0, 1)
    if x.dtype == KERNEL_DTYPE and x.is_cuda and x.stride(-1) == 1 and x.stride(0) % 128 == 0 \
            and x.stride(1) % 128 == 0 and x.data_ptr() % 16 == 0:
        return view
    return view.to(KERNEL_DTYPE).contiguous()


class T2TAttentionImpl(AttentionImpl):
    """Attention of one transformer layer (t2t_attn.py:1049-1080).  Rejects what
    the kernels do not implement: causal masks, head sizes other than 128,
    grouped-query attention and scales other than 1/sqrt(128)."""

    def __init__(self, num_heads: int, head_size: int, causal: bool, softmax_scale: float,
                 num_kv_heads: int | None = None, prefix: str = "", **extra_impl_args: Any) -> None:
        unsupported = (
            (bool(causal), "Token2Tile does not support causal attention"),
            (head_size != 128, "Token2Tile kernels require head dimension 128"),
            (num_kv_heads is not None and num_kv_heads != num_heads, "Token2Tile does not support grouped-query attention"),
            (not math.isclose(softmax_scale, 128 ** -0.5, rel_tol=1e-6), "Token2Tile has a fixed 1/sqrt(128) attention scale"),
        )
        for hit, message in unsupported:
            if hit:
                raise ValueError(message)
        self.num_heads, self.head_size, self.softmax_scale = num_heads, head_size, softmax_scale
        self.layer_idx = self._get_layer_idx(prefix)
        self._h3_states: dict[int, dict[str, torch.Tensor]] = {}
        self._dense = DenseAttention(num_heads, head_size, softmax_scale, num_kv_heads, prefix)

    @staticmethod
    def _get_layer_idx(prefix: str) -> int:
        """Index of the transformer block a module path belongs to
        (t2t_attn.py:1082-1090): the number after a "blocks" / "transformer_blocks"
        component, else the third component from the end."""
        parts = prefix.split(".")
        for name, nxt in zip(parts, parts[1:]):
            if name in ("blocks", "transformer_blocks") and nxt.isdigit():
                return int(nxt)
        if len(parts) < 3:
            raise ValueError(f"Invalid Token2Tile attention layer prefix: {prefix}")
        return int(parts[-3])

    # -- one CFG branch of one request: [1, N, H_local, 128] ---------------------
    def forward(self, query, key, value, attn_metadata: T2TAttentionMetadata):
        """Dense during the prefix steps, the sparse operator afterwards
        (t2t_attn.py:1092-1196).  The n-th call of a (step, layer) pair is CFG
        branch n; branch 0 may rebuild the structure, branch 1 reuses it."""
        if query.ndim != 4:
            raise ValueError("Token2Tile expects rank-4 SGL attention tensors")
        profile = resolve_profile(attn_metadata, int(query.shape[1]), self.num_heads)
        if attn_metadata.step_index < profile.dense_prefix_steps:
            return self._dense.forward(query, key, value)
        if query.shape != key.shape or query.shape != value.shape:
            raise ValueError("Token2Tile requires equal self-attention Q/K/V shapes")
        if query.shape[0] != 1:
            raise ValueError("Token2Tile currently requires one request/CFG branch per call")
        _, seq_len, heads, head_dim = query.shape
        ulysses = _ulysses_world_size()
        if self.num_heads % ulysses or heads != self.num_heads // ulysses or head_dim != self.head_size:
            raise ValueError("Token2Tile Q/K/V geometry changed after initialization: got "
                             f"H={heads} D={head_dim}, expected H={self.num_heads}/{ulysses} D={self.head_size}")
        if seq_len < max(profile.ck, profile.cq):
            raise ValueError("Token2Tile cluster count exceeds the token sequence length")

        runtime = _get_runtime(attn_metadata, profile, heads, seq_len, head_dim, query.device,
                               total_heads=self.num_heads)
        cache = attn_metadata.cache
        if cache.runtime_key is None:
            cache.runtime_key = runtime.key
        elif cache.runtime_key != runtime.key:
            raise RuntimeError("Token2Tile request geometry changed during denoising")
        if runtime.active_cache_id != id(cache):       # a new request: its snapshots start empty
            # the request boundary is also where the device status word of the previous request's calls is
            # examined: a kernel whose bounded wait gave up leaves garbage behind, and step() itself never syncs
            _check_operator_status(runtime.deploy)
            runtime.deploy.reset_cfg_reuse()
            runtime.active_cache_id = id(cache)
            cache.initialized_runtime = True

        call_key = (attn_metadata.step_index, self.layer_idx)
        parity = cache.call_counts.get(call_key, 0)
        if parity > 1:
            raise RuntimeError("Token2Tile observed more than two CFG branches for one layer/step")
        cache.call_counts[call_key] = parity + 1

        device = query.device
        # the host model runs under autocast; the operator's tensors keep their own types
        with torch.autocast(device_type=device.type, enabled=False):
            q, k, v = _heads_major(query[0]), _heads_major(key[0]), _heads_major(value[0])
            deploy = runtime.deploy
            _order_after_caller(deploy, device)
            deploy.set_cfg_call(parity, self.layer_idx, attn_metadata.step_index)
            ns = runtime.ns_map[(step_window(attn_metadata.step_index), self.layer_idx, parity)]
            _set_budget(deploy, runtime.ns_tensors[ns], device)
            state_key = (self.layer_idx, parity)
            state = cache.states.get(state_key)
            if state is None:
                state = deploy.init_state(q, k, warm_iters=attn_metadata.warm_iters,
                                          seed=self.layer_idx * 2 + parity)
                cache.states[state_key] = state
            previous = {name: state[name].clone() for name in ("ck", "cq")}
            if query.dtype == KERNEL_DTYPE and q.is_cuda and hasattr(deploy, "tile_attn_out"):
                # the operator writes its result straight into the host's [1, N, H, D] layout
                result = torch.empty_like(query)
                deploy.step(q, k, v, state, out=result[0].transpose(0, 1))
                _sanitize_state(state, previous)
                return result
            output = deploy.step(q, k, v, state)
            _sanitize_state(state, previous)
        return output.transpose(0, 1).unsqueeze(0).to(query.dtype).contiguous()

    @staticmethod
    def _current_step() -> int:
        context = _forward_context()
        return 0 if context is None else int(context.current_timestep)

    # -- packed [context | video | pad] document: [T, H_local, 128] ---------------
    def forward_varlen(self, query, key, value, *, cu_seqlens, max_seqlen: int, cu_seqlens_host=None):
        """Packed-document path of the 56-head model (t2t_attn.py:1209-1412).
        Context rows (text, audio, pinned condition frames) attend densely;
        video rows go through the operator with the context keys as one pinned,
        always-selected key cluster.  The operator needs as many queries as
        keys, so the first `context` video queries are repeated as padding and
        their outputs dropped.  bfloat16 has float32's exponent range, so the
        reference's fp16 overflow guard (|x| <= 8192, three host syncs per call)
        has nothing to guard here and is not run."""
        dense = lambda: self._dense.forward_varlen(query, key, value, cu_seqlens=cu_seqlens,
                                                   max_seqlen=max_seqlen, cu_seqlens_host=cu_seqlens_host)
        if self.num_heads != 56:
            return dense()
        step = self._current_step()
        cfg = _h3_config()
        if step < cfg["dense_prefix"]:
            return dense()
        used = int(max_seqlen)
        if used <= 0 or used > query.shape[0]:
            raise ValueError(f"Invalid H3 packed used length {used}/{query.shape[0]}")
        # The same backend also serves short auxiliary sequences (the prompt
        # refiner): anything that is not the main packed document stays dense.
        video_tokens, rows = cfg["video_tokens"], None
        from_layout, layout_rows = _h3_split(used, cfg["cond_mode"], query.device)
        if layout_rows is not None:
            video_tokens, rows = from_layout, layout_rows
        elif video_tokens <= 0:
            video_tokens = from_layout
        if video_tokens <= 0 or video_tokens >= used:
            return dense()
        local_heads = int(query.shape[1])
        ulysses = _ulysses_world_size()
        if local_heads * ulysses != self.num_heads:
            raise ValueError(f"H3 Token2Tile head sharding mismatch: local H={local_heads} x ulysses {ulysses} "
                             f"!= {self.num_heads}")
        heads_per_chunk = 28 if local_heads % 28 == 0 else local_heads
        num_chunks = local_heads // heads_per_chunk
        runtime = _get_h3_runtime(used, query.device, heads=heads_per_chunk, video_tokens=video_tokens)
        context, video = runtime.context_tokens, runtime.video_tokens
        if context > video:
            raise ValueError("H3 Token2Tile dummy query padding requires video >= context")
        deploy = runtime.deploy
        if step == runtime.dense_prefix:        # first sparse step of a request
            if cfg["persist_state"]:
                self._h3_states = {c: st for c, st in self._h3_states.items()
                                   if st["Uq"].shape[0] == heads_per_chunk and st["cq"].shape[1] == deploy.CQ
                                   and st["ck"].shape[1] == deploy.C}
            else:
                self._h3_states.clear()
            if self.layer_idx == 0:
                _check_operator_status(deploy)      # the previous request's calls: see forward()
                deploy.reset_cfg_reuse()

        device = query.device
        q_used, k_used, v_used = query[:used], key[:used], value[:used]
        qh, kh, vh = (t.transpose(0, 1) for t in (q_used, k_used, v_used))
        outputs = []
        with torch.autocast(device_type=device.type, enabled=False):
            for chunk in range(num_chunks):
                hs = slice(chunk * heads_per_chunk, (chunk + 1) * heads_per_chunk)
                if rows is None:
                    q_video = qh[hs, context:]
                    k_order = torch.cat((kh[hs, context:], kh[hs, :context]), dim=1)
                    v_order = torch.cat((vh[hs, context:], vh[hs, :context]), dim=1)
                else:
                    vid_rows, ctx_rows = rows
                    q_video = qh[hs].index_select(1, vid_rows)
                    k_order = torch.cat((kh[hs].index_select(1, vid_rows), kh[hs].index_select(1, ctx_rows)), dim=1)
                    v_order = torch.cat((vh[hs].index_select(1, vid_rows), vh[hs].index_select(1, ctx_rows)), dim=1)
                q_kernel = torch.cat((q_video, q_video[:, :context]), dim=1).to(KERNEL_DTYPE).contiguous()
                k_kernel = k_order.to(KERNEL_DTYPE).contiguous()
                v_kernel = v_order.to(KERNEL_DTYPE).contiguous()
                _order_after_caller(deploy, device)
                deploy.set_cfg_call(0, key=(self.layer_idx, chunk), step=step)
                ns = runtime.ns_map[(step_window(step), self.layer_idx)]
                _set_budget(deploy, runtime.ns_tensors[ns], device)
                state = self._h3_states.get(chunk)
                sync_init = cfg["sync_init"] and state is None and device.type == "cuda"
                if sync_init:
                    torch.cuda.synchronize(device)
                if state is None:
                    state = deploy.init_state(q_kernel, k_kernel, warm_iters=cfg["warm_iters"],
                                              seed=self.layer_idx * 8 + chunk)
                    self._h3_states[chunk] = state
                    if sync_init:
                        torch.cuda.synchronize(device)
                previous = {name: state[name].clone() for name in ("ck", "cq")}
                out = deploy.step(q_kernel, k_kernel, v_kernel, state)
                if sync_init:
                    torch.cuda.synchronize(device)
                _sanitize_state(state, previous)
                outputs.append(out[:, :video].float())

        video_output = torch.cat(outputs, dim=0).transpose(0, 1).to(query.dtype)
        context_q = q_used[:context] if rows is None else q_used.index_select(0, rows[1])
        context_output = self._dense.rows_over(context_q, k_used, v_used)
        result = torch.zeros_like(query)
        if rows is None:
            result[:context] = context_output
            result[context:used] = video_output
        else:
            result[rows[1]] = context_output
            result[rows[0]] = video_output
        if cfg["sync_first_sparse"] and step == runtime.dense_prefix and device.type == "cuda":
            torch.cuda.synchronize(device)
        return result
