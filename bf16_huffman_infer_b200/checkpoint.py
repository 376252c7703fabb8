"""Save and restore compressed models without re-encoding.

The reference re-compresses the model on every start: its compressed weights are ordinary module
buffers, so ``state_dict()`` already contains them (``<linear>.weight.{rem,exp,offsets,LUT1..4,
code_lengths}`` or ``.LUT``), but nothing rebuilds a :class:`CompressedLinear` from such a dictionary.
This module adds that step: ``save_compressed`` writes the state dict plus a small manifest of which
modules are compressed (and how), ``load_compressed`` swaps the matching ``nn.Linear`` modules of a
freshly constructed model for compressed ones and loads the buffers.
"""
from __future__ import annotations

from typing import Dict

import torch
from torch import nn

from .functional import (ANSWeight, CompressedLinear, FusedCompressedLinear, HuffmanWeight, _FusedSlice)

__all__ = ["save_compressed", "load_compressed", "compressed_manifest"]

_FORMAT = "bf16_huffman_infer_b200/1"


def _weight_meta(w: HuffmanWeight) -> Dict:
    return {"algo": w.algo, "rem": list(w.rem.shape), "exp": int(w.exp.numel()), "offsets": list(w.offsets.shape)}


def compressed_manifest(model: nn.Module) -> Dict:
    """Which modules of ``model`` are compressed, with the buffer shapes needed to rebuild them."""
    entries = {}
    for name, mod in model.named_modules():
        if isinstance(mod, CompressedLinear):
            entries[name] = {"kind": "linear", "bias": mod.bias is not None, **_weight_meta(mod.weight)}
        elif isinstance(mod, FusedCompressedLinear):
            entries[name] = {"kind": "fused", "bias": mod.bias is not None, "splits": [list(s) for s in mod.splits],
                             **_weight_meta(mod.weight)}
    slices = {}
    for name, mod in model.named_modules():
        if isinstance(mod, _FusedSlice):
            owner = next(n for n, m in model.named_modules() if m is mod._owner)
            slices[name] = {"owner": owner, "index": mod.index, "leader": mod.leader}
    return {"format": _FORMAT, "modules": entries, "slices": slices}


def save_compressed(model: nn.Module, path: str) -> None:
    """Write ``{"manifest": ..., "state_dict": ...}`` (CPU tensors) with ``torch.save``."""
    state = {k: v.detach().cpu() for k, v in model.state_dict().items()}
    torch.save({"manifest": compressed_manifest(model), "state_dict": state}, path)


def _empty_weight(meta: Dict) -> HuffmanWeight:
    rem = torch.empty(meta["rem"], dtype=torch.uint8)
    exp = torch.empty(meta["exp"], dtype=torch.int32)
    offsets = torch.empty(meta["offsets"], dtype=torch.int32)
    if meta["algo"] == "ans":
        return ANSWeight(rem, exp, offsets, torch.empty(256, dtype=torch.int32))
    tables = [torch.empty(256, dtype=torch.uint8) for _ in range(5)]
    return HuffmanWeight(rem, exp, offsets, *tables)


def load_compressed(model: nn.Module, path: str, strict: bool = True) -> nn.Module:
    """Turn ``model`` (same architecture, uncompressed, any initialisation) into the saved compressed
    model: the modules named in the manifest are replaced, then the state dict is loaded."""
    blob = torch.load(path, map_location="cpu", weights_only=False)
    manifest = blob["manifest"]
    if manifest.get("format") != _FORMAT:
        raise ValueError(f"not a compressed checkpoint of this package: {manifest.get('format')!r}")
    state = blob["state_dict"]
    owners = {}
    for name, meta in manifest["modules"].items():
        weight = _empty_weight(meta)
        if meta["kind"] == "linear":
            old = model.get_submodule(name)
            bias = nn.Parameter(torch.empty_like(old.bias), requires_grad=False) if meta["bias"] else None
            model.set_submodule(name, CompressedLinear(weight, bias))
        else:
            rows = meta["splits"][-1][1]
            bias = nn.Parameter(torch.empty(rows, dtype=state[name + ".bias"].dtype), requires_grad=False) if meta["bias"] else None
            owners[name] = FusedCompressedLinear(weight, bias, [tuple(s) for s in meta["splits"]])
    for name, info in manifest["slices"].items():
        model.set_submodule(name, _FusedSlice(owners[info["owner"]], info["index"], info["leader"]))
    model.load_state_dict(state, strict=strict)
    return model
