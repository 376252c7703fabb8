"""Save and restore compressed models without re-encoding.

The reference re-compresses the model on every start: its compressed weights are ordinary module
buffers, so ``state_dict()`` already contains them (``<linear>.weight.{rem,exp,offsets,LUT1..4,
code_lengths}`` or ``.LUT``), but nothing rebuilds a :class:`CompressedLinear` from such a dictionary.
This module adds that step: ``save_compressed`` writes the state dict plus a small manifest of which
modules are compressed (and how), ``load_compressed`` swaps the matching ``nn.Linear`` modules of a
freshly constructed model for compressed ones and loads the buffers.

On disk: one ``safetensors`` file - the format's tensors under their state-dict names, the manifest as a
JSON string in the file's metadata.  Nothing is unpickled on load, and the manifest is checked against
the model it is applied to (module names, layer shapes) before any module is replaced.
"""
from __future__ import annotations

import json
from typing import Dict

import torch
from safetensors import safe_open
from safetensors.torch import save_file
from torch import nn

from .functional import (ANSWeight, CompressedLinear, FusedCompressedLinear, HuffmanWeight, _FusedSlice)

__all__ = ["save_compressed", "load_compressed", "compressed_manifest"]

_FORMAT = "bf16_huffman_infer_b200/1"


def _weight_meta(w: HuffmanWeight) -> Dict:
    meta = {"algo": w.algo, "rem": list(w.rem.shape), "exp": int(w.exp.numel()), "offsets": list(w.offsets.shape)}
    if w.algo == "ans":
        meta["lut"] = int(w.LUT.numel())        # 2^precision table words
    return meta


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
    """Write the state dict (CPU tensors) as a safetensors file with the manifest in its metadata."""
    state = {}
    seen = {}
    for k, v in model.state_dict().items():
        t = v.detach().cpu().contiguous()
        # safetensors refuses tensors that share storage (tied embeddings): store such a tensor once more
        state[k] = t.clone() if t.data_ptr() in seen else t
        seen[t.data_ptr()] = k
    save_file(state, path, metadata={"manifest": json.dumps(compressed_manifest(model))})


def _validate(model: nn.Module, manifest: Dict) -> None:
    """The manifest must describe THIS model: every named module exists and is a linear layer of the shape the
    compressed buffers encode (``rem`` is ``[S, out_features, in_features / S]``)."""
    def check_shape(name: str, meta: Dict, out_features: int, in_features: int) -> None:
        rem = meta.get("rem")
        if (meta.get("algo") not in ("huffman", "ans") or not isinstance(rem, list) or len(rem) != 3
                or rem[1] != out_features or rem[0] * rem[2] != in_features
                or meta.get("offsets") != [rem[0], rem[1]] or not isinstance(meta.get("exp"), int) or meta["exp"] < 64
                or meta.get("lut", 256) not in (256, 512, 1024, 2048, 4096)):
            raise ValueError(f"checkpoint entry {name!r} does not fit a linear layer {in_features} -> {out_features}: {meta}")

    names = dict(model.named_modules())
    for name, meta in manifest.get("modules", {}).items():
        if meta.get("kind") == "linear":
            old = names.get(name)
            if not isinstance(old, nn.Linear):
                raise ValueError(f"checkpoint names {name!r}, which is not an nn.Linear of this model")
            check_shape(name, meta, old.out_features, old.in_features)
        elif meta.get("kind") == "fused":
            members = sorted((info["index"], n) for n, info in manifest.get("slices", {}).items() if info.get("owner") == name)
            splits = meta.get("splits")
            if not members or not isinstance(splits, list) or [i for i, _ in members] != list(range(len(splits))):
                raise ValueError(f"stacked entry {name!r} has no consistent set of slices")
            olds = [names.get(n) for _, n in members]
            if not all(isinstance(o, nn.Linear) for o in olds):
                raise ValueError(f"a slice of {name!r} is not an nn.Linear of this model")
            if [list(sp) for sp in splits] != [[sum(o.out_features for o in olds[:i]), sum(o.out_features for o in olds[:i + 1])]
                                               for i in range(len(olds))] or len({o.in_features for o in olds}) != 1:
                raise ValueError(f"stacked entry {name!r} does not match the layers it replaces")
            check_shape(name, meta, splits[-1][1], olds[0].in_features)
        else:
            raise ValueError(f"unknown entry kind in checkpoint: {meta.get('kind')!r}")


def _empty_weight(meta: Dict) -> HuffmanWeight:
    rem = torch.empty(meta["rem"], dtype=torch.uint8)
    exp = torch.empty(meta["exp"], dtype=torch.int32)
    offsets = torch.empty(meta["offsets"], dtype=torch.int32)
    if meta["algo"] == "ans":
        return ANSWeight(rem, exp, offsets, torch.empty(int(meta.get("lut", 256)), dtype=torch.int32))
    tables = [torch.empty(256, dtype=torch.uint8) for _ in range(5)]
    return HuffmanWeight(rem, exp, offsets, *tables)


def load_compressed(model: nn.Module, path: str, strict: bool = True) -> nn.Module:
    """Turn ``model`` (same architecture, uncompressed, any initialisation) into the saved compressed
    model: the modules named in the manifest are replaced, then the state dict is loaded."""
    with safe_open(path, framework="pt", device="cpu") as f:
        meta = f.metadata() or {}
        if "manifest" not in meta:
            raise ValueError("not a compressed checkpoint of this package: no manifest in the file's metadata")
        manifest = json.loads(meta["manifest"])
        if not isinstance(manifest, dict) or manifest.get("format") != _FORMAT:
            raise ValueError(f"not a compressed checkpoint of this package: {manifest.get('format') if isinstance(manifest, dict) else manifest!r}")
        state = {k: f.get_tensor(k) for k in f.keys()}
    _validate(model, manifest)
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
