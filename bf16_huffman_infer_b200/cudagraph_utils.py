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
"""
from __future__ import annotations

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


def apply_graphed(model: nn.Module, cache, replace_generate: bool = True) -> None:
    """Swap ``model.forward`` (and ``model.generate``) for the graph-replaying versions, in place."""
    old_forward = model.forward
    graphs: Dict[int, _StepGraph] = {}

    def forward(input_ids: Optional[torch.LongTensor] = None, attention_mask=None, position_ids=None,
                past_key_values=None, inputs_embeds=None, **kwargs) -> CausalLMOutputWithPast:
        one_token = (input_ids is not None and input_ids.dim() == 2 and input_ids.shape[1] == 1 and input_ids.is_cuda
                     and attention_mask is None and position_ids is None and inputs_embeds is None
                     and not torch.is_grad_enabled())
        if one_token:
            batch = input_ids.shape[0]
            step = graphs.get(batch)
            if step is None and _room_for_capture(cache):
                step = graphs[batch] = _StepGraph(old_forward, cache, batch, input_ids.device)
            if step is not None:
                return CausalLMOutputWithPast(logits=step(input_ids), past_key_values=cache)
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
            with torch.no_grad():
                return old_generate(*args, past_key_values=cache, disable_compile=True, **kwargs)

        model.generate = generate


def get_graphed_model(model: nn.Module, cache) -> nn.Module:
    """A copy of ``model`` (sharing its weights) whose one-token steps replay a CUDA graph."""
    graphed = shallow_copy_model(model)
    apply_graphed(graphed, cache)
    return graphed
