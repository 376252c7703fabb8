"""CUDA-graph the one-token decode step of a Hugging Face causal LM that uses a ``StaticCache``.

Same entry points and contract as the reference's ``bf16_huffman_infer/cudagraph_utils.py``
(``apply_graphed`` :11-80, ``get_graphed_model`` :83-86): the returned model shares all parameters
and buffers with the original, runs every call with a single new token per sequence through a
captured CUDA graph, runs everything else (the prompt) eagerly, and its ``generate`` resets the
cache and decodes into it.

What differs is how the step is captured.  The reference graphs a closure over four tensors
(ids, a 4-D float mask, position ids, cache position) for batch 1 only; with the transformers
release this package targets (5.x) the static cache keeps its fill level in a device tensor and
the model derives positions and masks from it, so the captured step takes the token ids alone and
works for any batch size the cache was built for.  Graphs are captured lazily, one per batch size,
the first time a one-token step of that size is seen (i.e. after the prompt has been processed,
when the cache tensors exist).

``generate`` hands every step an attention mask and position ids.  Without padding both carry no
information beyond the cache's fill level (the mask is all ones, every sequence sits at the same
position), so the captured step - which lets the model derive them from the cache - is used
whenever the mask of the call is all ones; the check is made once per ``generate`` call on the
mask the caller passed.  A batch with padding runs eagerly (with a one-time warning).  How often
each path ran is kept in ``model.graph_stats``.
"""
from __future__ import annotations

import warnings
from typing import Dict, Optional

import torch
from torch import nn
from transformers.modeling_outputs import CausalLMOutputWithPast

from .utils import shallow_copy_model

__all__ = ["apply_graphed", "get_graphed_model"]

_WARMUP_STEPS = 2


class _StepGraph:
    """One captured decode step for a fixed batch size."""

    def __init__(self, forward, cache, batch: int, device: torch.device):
        self.ids = torch.zeros(batch, 1, dtype=torch.int64, device=device)
        fills = [layer.cumulative_length for layer in cache.layers if hasattr(layer, "cumulative_length")]
        saved = [f.clone() for f in fills]

        def step():
            return forward(input_ids=self.ids, past_key_values=cache, use_cache=True, return_dict=True).logits

        # Warm-up and capture advance the cache's fill level and write a few slots past it; the
        # level is put back afterwards and those slots are rewritten by the real tokens later.
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(_WARMUP_STEPS):
                step()
        torch.cuda.current_stream(device).wait_stream(side)
        for f, s in zip(fills, saved):
            f.copy_(s)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.logits = step()
        for f, s in zip(fills, saved):
            f.copy_(s)

    def __call__(self, input_ids: torch.Tensor) -> torch.Tensor:
        self.ids.copy_(input_ids)
        self.graph.replay()
        return self.logits.clone()


def _room_for_capture(cache) -> bool:
    """Capturing writes ``_WARMUP_STEPS + 1`` slots past the current fill level; they must exist."""
    for layer in cache.layers:
        if not getattr(layer, "is_initialized", False):
            return False
        if int(layer.cumulative_length.item()) + _WARMUP_STEPS + 1 > layer.max_cache_len:
            return False
    return True


def _all_ones(mask) -> Optional[bool]:
    """True / False for a 2-D mask tensor (costs a synchronisation), None for forms that are not inspected."""
    if mask is None:
        return True
    if torch.is_tensor(mask) and mask.dim() == 2:
        return bool(mask.all())
    return None


def apply_graphed(model: nn.Module, cache, replace_generate: bool = True) -> None:
    """Swap ``model.forward`` (and ``model.generate``) for the graph-replaying versions, in place."""
    old_forward = model.forward
    graphs: Dict[int, _StepGraph] = {}
    stats = {"captures": 0, "replays": 0, "eager_steps": 0}
    model.graph_stats = stats
    # None outside generate(); inside: whether the mask the caller passed was free of padding
    state = {"no_padding": None, "warned": False}

    def trivial_inputs(attention_mask, position_ids) -> bool:
        if state["no_padding"] is not None:
            return state["no_padding"]
        if attention_mask is None and position_ids is None:
            return True
        # a direct call with a mask: inspect it (a synchronisation); position ids cannot be checked cheaply
        return position_ids is None and _all_ones(attention_mask) is True

    def forward(input_ids: Optional[torch.LongTensor] = None, attention_mask=None, position_ids=None,
                past_key_values=None, inputs_embeds=None, **kwargs) -> CausalLMOutputWithPast:
        one_token = (input_ids is not None and input_ids.dim() == 2 and input_ids.shape[1] == 1 and input_ids.is_cuda
                     and inputs_embeds is None and not torch.is_grad_enabled())
        if one_token and trivial_inputs(attention_mask, position_ids):
            batch = input_ids.shape[0]
            step = graphs.get(batch)
            if step is None and _room_for_capture(cache):
                step = graphs[batch] = _StepGraph(old_forward, cache, batch, input_ids.device)
                stats["captures"] += 1
            if step is not None:
                stats["replays"] += 1
                return CausalLMOutputWithPast(logits=step(input_ids), past_key_values=cache)
        if one_token:
            stats["eager_steps"] += 1
            if not state["warned"]:
                state["warned"] = True
                warnings.warn("one-token step run eagerly: the batch has padding (or explicit position ids), "
                              "which the captured CUDA graph does not take as inputs")
        kwargs.pop("use_cache", None)
        kwargs.pop("return_dict", None)
        return old_forward(input_ids=input_ids, attention_mask=attention_mask, position_ids=position_ids,
                           past_key_values=cache, inputs_embeds=inputs_embeds, use_cache=True, return_dict=True, **kwargs)

    model.forward = forward

    if replace_generate:
        old_generate = model.generate

        def generate(*args, **kwargs):
            cache.reset()
            kwargs.pop("past_key_values", None)
            verdict = _all_ones(kwargs.get("attention_mask"))
            if kwargs.get("attention_mask") is None:
                # generate() derives a mask from pad tokens in the prompt when it is given none
                ids = kwargs.get("input_ids", args[0] if args else None)
                pad = getattr(getattr(model, "generation_config", None), "pad_token_id", None)
                if torch.is_tensor(ids) and pad is not None and bool((ids == pad).any()):
                    verdict = False
            state["no_padding"] = bool(verdict)          # uninspectable forms count as padded
            try:
                with torch.no_grad():
                    return old_generate(*args, past_key_values=cache, disable_compile=True, **kwargs)
            finally:
                state["no_padding"] = None

        model.generate = generate


def get_graphed_model(model: nn.Module, cache) -> nn.Module:
    """A copy of ``model`` (sharing its weights) whose one-token steps replay a CUDA graph."""
    graphed = shallow_copy_model(model)
    apply_graphed(graphed, cache)
    return graphed
