"""convert(model, policy) / calibrate(model, data): per-layer precision routing
(API of src/thor_fp4/convert.py:29-188 in the reference project).

policy: "auto" (shape table / crossover rule), "fp4", "mx8", "bf16", a dict of
fnmatch patterns -> spec (first match wins, unmatched -> "auto"), or a callable
(name, module) -> spec.  The decision per layer is recorded in
``model.thor_fp4_policy``.
"""
from __future__ import annotations

import copy
import fnmatch
import json
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.nn as nn

from .linear import Linear

__all__ = ["convert", "calibrate", "auto_decision", "load_shape_table", "shape_table_path"]

_TABLE = Path(__file__).resolve().parent / "shape_table.json"
_FALLBACK = {"min_k": 2048, "min_n": 512}


def shape_table_path() -> Path:
    return _TABLE


def load_shape_table() -> dict:
    if _TABLE.exists():
        return json.loads(_TABLE.read_text())
    return {"crossover": dict(_FALLBACK), "shapes": {}}


@dataclass
class Decision:
    spec: str      # "fp4" | "bf16"
    reason: str


def auto_decision(in_features: int, out_features: int, table: dict | None = None) -> Decision:
    """Shape-aware FP4 / BF16 choice for a (K=in, N=out) layer: hard constraints first,
    then a measured table row ("<N>x<K>"), then the crossover rule."""
    table = table or load_shape_table()
    K, N = in_features, out_features
    if K % 64 != 0:
        return Decision("bf16", f"K={K} not a multiple of 64 (scale tiles are 4 sf wide)")
    if N < 8 or N % 8 != 0:
        return Decision("bf16", f"N={N} violates the GEMM's N>=8, N%8==0 constraint")
    entry = table.get("shapes", {}).get(f"{N}x{K}")
    if entry is not None:
        row = entry if "fp4_ms" in entry else (entry.get("4096") or next(iter(entry.values())))
        return Decision("fp4" if row.get("fp4_wins", False) else "bf16",
                        f"measured: fp4 {row['fp4_ms']:.4f} ms vs bf16 {row['bf16_ms']:.4f} ms "
                        "(quantize included)")
    cross = table.get("crossover", _FALLBACK)
    if K >= cross["min_k"] and N >= cross["min_n"]:
        return Decision("fp4", f"K={K} >= {cross['min_k']} and N={N} >= {cross['min_n']} (measured crossover)")
    return Decision("bf16", f"K={K} < {cross['min_k']} or N={N} < {cross['min_n']} "
                            "(small-K shapes: FP4 kernels lose to BF16)")


def _match_policy(policy, name: str, module: nn.Module):
    if isinstance(policy, str):
        return policy
    if callable(policy):
        return policy(name, module)
    if isinstance(policy, dict):
        for pat, spec in policy.items():
            if name == pat or fnmatch.fnmatch(name, pat):
                return spec
        return "auto"
    raise TypeError(f"bad policy: {policy!r}")


def _swap(root: nn.Module, name: str, new: nn.Module):
    parent, _, attr = name.rpartition(".")
    setattr(root.get_submodule(parent) if parent else root, attr, new)


@torch.no_grad()
def convert(model: nn.Module, policy="auto", calibration: dict | None = None,
            out_dtype: str = "f16", inplace: bool = False) -> nn.Module:
    """Replace nn.Linear layers by thor_fp4.Linear according to `policy`; `calibration`
    maps module names to static activation scales (from calibrate()).  Returns a deep
    copy unless inplace=True."""
    model = model if inplace else copy.deepcopy(model)
    table = load_shape_table()
    decisions: dict[str, str] = {}
    todo: list[tuple[str, nn.Linear, str]] = []
    for name, m in model.named_modules():
        if not isinstance(m, nn.Linear):
            continue
        spec = _match_policy(policy, name, m)
        engine = "cublaslt"
        if spec == "auto":
            spec = auto_decision(m.in_features, m.out_features, table).spec
        decisions[name] = spec
        if spec == "mx8":
            from .linear import resolve_mx8_variant
            try:
                if m.in_features % 128 != 0:
                    raise ValueError(f"K={m.in_features} not a multiple of 128")
                engine = f"cutlass:{resolve_mx8_variant(m.in_features)}"
                decisions[name] = "mx8: FP4 weights x MXFP8 acts (quality policy)"
            except (RuntimeError, ValueError) as e:
                fb = auto_decision(m.in_features, m.out_features, table)
                decisions[name] = f"mx8-unavailable ({e}); {fb.spec}: {fb.reason}"
                spec = fb.spec
        if spec in ("fp4", "mx8"):
            todo.append((name, m, engine))
    for name, m, engine in todo:
        try:
            new = Linear(m.in_features, m.out_features, bias=m.bias is not None,
                         out_dtype=out_dtype, device=m.weight.device, engine=engine)
        except ValueError as e:
            decisions[name] = f"bf16 ({e})"
            continue
        new.weight.copy_(m.weight.detach().float())
        if m.bias is not None:
            new.bias.copy_(m.bias.detach().float())
        if calibration and name in calibration:
            new.act_tensor_scale = float(calibration[name])
        _swap(model, name, new)
    model.thor_fp4_policy = decisions
    return model


@torch.no_grad()
def calibrate(model: nn.Module, sample_inputs) -> dict:
    """Running amax of every nn.Linear's input over the calibration batches ->
    {module name: amax / (6*448)}.  sample_inputs: a batch, a list of batches, or a
    callable yielding batches."""
    amax: dict[str, float] = {}
    hooks = []
    for name, m in model.named_modules():
        if isinstance(m, nn.Linear):
            def hook(mod, inp, out, _name=name):
                amax[_name] = max(amax.get(_name, 0.0), inp[0].abs().amax().item())
            hooks.append(m.register_forward_hook(hook))
    try:
        batches = sample_inputs() if callable(sample_inputs) else (
            sample_inputs if isinstance(sample_inputs, list) else [sample_inputs])
        for b in batches:
            model(b)
    finally:
        for h in hooks:
            h.remove()
    return {n: a / (6.0 * 448.0) for n, a in amax.items()}
