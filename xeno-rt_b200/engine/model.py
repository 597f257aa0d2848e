"""A model instance: the parts that a ``ModelSpec`` names, built with their weights on one device.

Plays the role of ``LlamaModel::from_gguf`` (crates/xrt-models/src/llama.rs:297-378): read the
configuration, bind the tensors by name, prepare what the forward pass needs.  Unlike the
reference, shapes are checked at load and the model is assembled from registered parts.
"""
from __future__ import annotations

import dataclasses

import torch

from ..cache import Cache, KVNeed
from ..config import config_from_dict, load_config
from ..core import DType, KernelError, log, parse_dtype, torch_dtype
from ..csrc import ops
from ..parts import LayerParts, ModelSpec, part_class
from ..weights import (INIT_MATRIX_STD, INIT_NORM_STD, load_weights, tensor_key)
from ..weights.loader import LoadedTensors, kept_dtype


class Model:
    def __init__(self, spec: ModelSpec, tensors: dict, dtype: DType, device, config=None):
        ops.require_device()
        spec.validate()
        self.spec = spec
        self.config = config
        self.dtype = dtype
        self.device = torch.device(device)
        self.vocab_size = spec.vocab_size
        self.hidden_size = spec.hidden_size
        self.max_positions = spec.max_positions

        shared = getattr(tensors, "fused", {})

        def build(role, part_spec):
            cls = part_class(role, part_spec.kind)
            weights = {r: tensors[name] for r, name in part_spec.weights.items()}
            fused = getattr(cls, "fused_weights", None)
            for fused_role, roles in (fused(part_spec.params).items() if fused else ()):
                buffer = shared.get(tuple(part_spec.weights[r] for r in roles))
                if buffer is not None:  # the loader put these tensors side by side already
                    weights[fused_role] = buffer
            return cls(part_spec.params, weights, dtype, self.device)

        self.embedding = build("embedding", spec.embedding)
        self.layers = [LayerParts({name: build(role, part) for name, (role, part) in l.parts.items()},
                                  {name: role for name, (role, _) in l.parts.items()}) for l in spec.layers]
        self.arrangements = [part_class("arrangement", l.arrangement) for l in spec.layers]
        self.final_norm = build("norm", spec.final_norm)
        self.lm_head = build("lm_head", spec.lm_head)
        self.error_flag = ops.device_state(self.device)[0]
        parts = [self.embedding, self.final_norm, self.lm_head]
        for layer in self.layers:
            parts += list(layer.values())
        self.graph_safe = all(getattr(p, "graph_safe", False) for p in parts)
        # what each place of the schedule is followed by: the first norm of the layer that runs next and
        # the part that takes its result, for arrangements that say so (see parts/block.py)
        firsts = [getattr(fn, "first_norm", None) for fn in self.arrangements]
        order = [firsts[place.layer](self.layers[place.layer]) if firsts[place.layer] else None
                 for place in spec.schedule]
        self._next_layer = order[1:] + [None]

    # ------------------------------------------------------------------ construction
    @classmethod
    def load(cls, folder: str, dtype="bfloat16", device="cuda:0") -> "Model":
        """From a folder with config.json and model.safetensors; the model class is chosen by
        config.json's architecture name."""
        ops.require_device()
        dtype = parse_dtype(dtype)
        arch, config = load_config(folder)
        spec = arch.build_spec(config)
        tensors = load_weights(folder, spec.expected_tensors(), dtype, device, spec.ignorable_tensors,
                               fused_groups=spec.fused_groups())
        log("info", f"loaded {arch.name} from {folder}: {len(spec.layers)} layers, width {spec.hidden_size}, "
                    f"vocabulary {spec.vocab_size}, {dtype.label}")
        return cls(spec, tensors, dtype, device, config)

    @classmethod
    def random(cls, config, seed: int = 0, dtype="bfloat16", device="cuda:0") -> "Model":
        """Random weights drawn on the device from ``seed`` with the generator of
        weights/random_init.py, without a model folder (for models of many gigabytes)."""
        ops.require_device()
        dtype = parse_dtype(dtype)
        raw = config if isinstance(config, dict) else config.to_dict()
        arch, typed = config_from_dict(raw)
        spec = arch.build_spec(typed)
        tensors = LoadedTensors()
        expected = {e.name: e for e in spec.expected_tensors()}
        for group in spec.fused_groups():  # one buffer for tensors that a part wants side by side
            members = [expected[n] for n in group]
            buffer = torch.empty((sum(e.shape[0] for e in members),) + tuple(members[0].shape[1:]),
                                 dtype=kept_dtype(members[0].kind, torch_dtype(dtype), dtype), device=device)
            begin = 0
            for e in members:
                tensors[e.name] = buffer[begin:begin + e.shape[0]]
                begin += e.shape[0]
            tensors.fused[tuple(group)] = buffer
        for e in expected.values():
            t = tensors.get(e.name)
            if t is None:
                t = torch.empty(e.shape, dtype=kept_dtype(e.kind, torch_dtype(dtype), dtype), device=device)
            if e.kind == "vector":
                ops.fill_normal(t, tensor_key(seed, e.name), 1.0, INIT_NORM_STD)
            else:
                ops.fill_normal(t, tensor_key(seed, e.name), 0.0, INIT_MATRIX_STD)
            tensors[e.name] = t
        return cls(spec, tensors, dtype, device, typed)

    # ------------------------------------------------------------------ cache
    def _layer_needs(self, layer: LayerParts) -> dict:
        """{part name: what the part asks of the cache} for the parts of a layer that ask for any
        (``cache_need()`` returning a KVNeed, a StateNeed or a list of them)."""
        needs = {}
        for name in layer.names():
            ask = getattr(layer[name], "cache_need", None)
            need = ask() if ask is not None else None
            if need is not None:
                needs[name] = need
        return needs

    def cache_needs(self) -> list:
        """One entry for each place of the schedule: what the parts of its layer ask of the cache,
        by part name, or None for a place that reads another place's storage."""
        needs = []
        for place in self.spec.schedule:
            needs.append(None if place.cache_from is not None else self._layer_needs(self.layers[place.layer]))
        # A place that reads another place's keys may see further back than the owner does: the
        # storage keeps the widest window of all its users (None = every key).
        for place in self.spec.schedule:
            if place.cache_from is None:
                continue
            for name, reader in self._layer_needs(self.layers[place.layer]).items():
                owner = needs[place.cache_from].get(name)
                if isinstance(owner, KVNeed) and isinstance(reader, KVNeed) and owner.window is not None:
                    wider = None if reader.window is None else max(owner.window, reader.window)
                    needs[place.cache_from][name] = dataclasses.replace(owner, window=wider)
        return needs

    def new_cache(self, max_tokens: int, max_slots: int | None = None) -> Cache:
        return Cache(self.cache_needs(), max_tokens, self.max_positions, self.dtype, self.device, max_slots)

    # ------------------------------------------------------------------ forward
    def forward(self, ctx, cache: Cache, want_rows: torch.Tensor | None):
        """Runs the tokens of ``ctx`` through every place of the schedule and returns float32
        logits [len(want_rows), vocab] (None if no row is wanted).  The order inside is that of
        crates/xrt-models/src/llama.rs:432-613; the final norm and the output matrix see only the
        wanted rows (llama.rs:814-819 does so for the last token)."""
        x = self.embedding.forward(ctx.token_ids, self.error_flag)
        for i, place in enumerate(self.spec.schedule):
            owns = place.cache_from is None
            stores = cache.store(i if owns else place.cache_from) or {}
            ctx.shared["next_layer"] = self._next_layer[i]
            self.arrangements[place.layer](self.layers[place.layer], x, ctx, stores, owns)
        ctx.pending = ctx.then_norm = None
        if want_rows is None or want_rows.numel() == 0:
            return None
        return self.lm_head.forward(self.final_norm.forward(x, want_rows))
