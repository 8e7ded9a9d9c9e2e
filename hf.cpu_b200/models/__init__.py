"""A model put together from a plan: parts per layer, the run order, weights bound by name.

``Model.forward`` is the forward pass the step function drives: embedding, the schedule's
entries in order, then the final norm and the head on the rows whose logits are wanted
(src/model.c:545-640).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from ..config import ModelConfig, load_config
from ..config.base import ModelPlan
from ..parts import make_part
from ..weights import RandomSource, TensorSpec, load_tensors


@dataclass
class Layer:
    block: object
    norm1: object
    mixer: object
    norm2: object
    ffn: object

    def parts(self):
        return (self.block, self.norm1, self.mixer, self.norm2, self.ffn)


class Model:
    def __init__(self, config: ModelConfig, run_dtype: torch.dtype = torch.bfloat16,
                 device: torch.device = torch.device("cuda:0"), plan: Optional[ModelPlan] = None):
        if run_dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"run dtype must be bfloat16 or float32, got {run_dtype}")
        self.config, self.run_dtype, self.device = config, run_dtype, torch.device(device)
        self.plan = plan if plan is not None else config.plan()
        self.plan.validate()
        p = self.plan
        self.positions = {name: make_part("position", spec) for name, spec in p.positions.items()}
        self.embedding = make_part("embedding", p.embedding)
        self.layers: List[Layer] = []
        for ls in p.layers:
            self.layers.append(Layer(
                block=make_part("block", ls.block),
                norm1=make_part("norm", ls.norm1),
                mixer=make_part("mixer", ls.mixer, positions=self.positions),
                norm2=make_part("norm", ls.norm2),
                ffn=make_part("ffn", ls.ffn)))
        self.final_norm = make_part("norm", p.final_norm)
        self.head = make_part("head", p.head)
        self.bound = False
        self.files: List[str] = []            # the weight files this model was loaded from

    # ---- weights ------------------------------------------------------------------------
    def all_parts(self):
        yield self.embedding
        yield from self.positions.values()
        for l in self.layers:
            yield from l.parts()
        yield self.final_norm
        yield self.head

    def tensor_specs(self) -> List[TensorSpec]:
        seen: Dict[str, TensorSpec] = {}
        for part in self.all_parts():
            for s in part.tensor_specs():
                if s.name in seen and seen[s.name].shape != s.shape:
                    raise ValueError(f"tensor '{s.name}' is declared with two shapes")
                seen.setdefault(s.name, s)
        return list(seen.values())

    def bind(self, tensors) -> "Model":
        """Hand the weights to the parts.  ``tensors`` maps names to tensors: a dict, or a source that makes
        each tensor when it is asked for, so that the parts take them one at a time."""
        if hasattr(tensors, "keep"):
            # a tensor that two parts bind (a tied head reads the embedding) is made once
            count: Dict[str, int] = {}
            for part in self.all_parts():
                for s in part.tensor_specs():
                    count[s.name] = count.get(s.name, 0) + 1
            tensors.keep(n for n, c in count.items() if c > 1)
        for part in self.all_parts():
            part.bind(tensors, self.run_dtype, self.device)
        for pos in self.positions.values():
            pos.prepare(self.plan.max_positions, self.device)
        self.bound = True
        return self

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights one decode step reads: every schedule entry's layer and the head, once each."""
        total = self.head.weight_bytes() + self.final_norm.weight_bytes()
        for e in self.plan.schedule:
            total += sum(p.weight_bytes() for p in self.layers[e.layer].parts())
        return total

    # ---- forward ------------------------------------------------------------------------
    def forward(self, ctx) -> Optional[torch.Tensor]:
        T = ctx.token_ids.shape[0]
        x = ctx.buf("residual", (T, self.plan.hidden_size), torch.float32)
        self.embedding.forward(ctx.token_ids, x)
        schedule = self.plan.schedule
        xn = None                                # norm1 of the coming block, when the previous block computed it
        for i, e in enumerate(schedule):
            layer = self.layers[e.layer]
            owner = i if e.cache_of is None else e.cache_of
            # the norm that follows this block: the next block's first, or, after the last block of a step whose
            # tokens all want their logits (a step of single tokens), the final norm
            if i + 1 < len(schedule):
                next_norm = self.layers[schedule[i + 1].layer].norm1
            else:
                next_norm = self.final_norm if getattr(ctx, "logits_for_all", False) else None
            xn = layer.block.forward(ctx, x, layer.norm1, layer.mixer, layer.norm2, layer.ffn,
                                     ctx.entry_cache(owner), ctx.entry_state(i), e.cache_of is None,
                                     xn_ready=xn, next_norm=next_norm)
        M = ctx.num_logit_rows
        if M == 0:
            return None
        if xn is None or not schedule:
            xn = ctx.buf("head_xn", (M, self.plan.hidden_size), self.run_dtype)
            self.final_norm.forward(x, xn, rows=ctx.logit_rows)
        logits = ctx.buf("logits", (M, self.plan.vocab_size), torch.float32)
        self.head.forward(xn, logits)
        return logits


def build_model_specs(config: ModelConfig) -> List[TensorSpec]:
    return Model(config, torch.float32, torch.device("cpu")).tensor_specs()


def load_model(path: str, dtype: torch.dtype = torch.bfloat16, device="cuda:0") -> Model:
    """Load a model folder (``config.json`` + safetensors: one file, or shards with or without an index) or one of
    the reference's GGUF files; the model class follows the configuration.  Every tensor is checked against the
    model's declaration before any is read, and tensors go to the device one at a time."""
    if os.path.isfile(path) and path.endswith(".gguf"):
        return load_gguf_model(path, dtype, device)
    config = load_config(path)
    model = Model(config, dtype, torch.device(device))
    tensors = load_tensors(path, model.tensor_specs(), dtype, model.device)
    try:
        model.bind(tensors)
        model.files = tensors.paths()
    finally:
        tensors.close()
    return model


def load_gguf_model(path: str, dtype: torch.dtype = torch.bfloat16, device="cuda:0") -> Model:
    """The same from one of the reference's own GGUF files (float tensor types only)."""
    from ..weights.gguf import GgufSource
    tensors = GgufSource(path, dtype, torch.device(device))
    try:
        model = Model(tensors.config, dtype, torch.device(device))
        tensors.check(model.tensor_specs())
        model.bind(tensors)
        model.files = [path]
    finally:
        tensors.close()
    return model


def random_model(config: ModelConfig, seed: int = 0, dtype: torch.dtype = torch.bfloat16, device="cuda:0",
                 std: float = 0.02) -> Model:
    """A model with random weights made directly on ``device`` (no files), one tensor at a time."""
    model = Model(config, dtype, torch.device(device))
    store = torch.float32 if dtype == torch.float32 else torch.bfloat16
    return model.bind(RandomSource(model.tensor_specs(), seed, store, model.device, std=std))
