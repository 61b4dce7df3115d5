"""The model: parts assembled from a ``ModelSpec``, and nothing else.

``Model`` builds the embedding, one block per ``LayerSpec``, the final norm and
the head through the part registries, gathers the tensors they need under their
full names, and hands loaded tensors back to them.  The order in which layers
run is ``spec.schedule``.
"""

from __future__ import annotations

import torch

from ..config.spec import ModelSpec
from ..parts import Runtime, WeightSpec, build_part


class Model:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        self.spec, self.rt = spec, runtime
        self.embedding = build_part("embedding", spec.embedding, runtime)
        self.blocks = [build_part("block", layer.block, runtime, layer_spec=layer) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.head = build_part("head", spec.head, runtime)
        self.tied_head = bool(getattr(self.head, "tied", False))

    # -- weights ------------------------------------------------------------
    def _named_parts(self):
        n = self.spec.names
        yield n["embedding"], self.embedding
        for layer, block in zip(self.spec.layers, self.blocks):
            yield layer.prefix, block
        yield n["final_norm"], self.final_norm
        yield n["head"], self.head

    def weight_specs(self) -> dict[str, WeightSpec]:
        out: dict[str, WeightSpec] = {}
        for prefix, part in self._named_parts():
            for local, spec in part.weight_specs().items():
                out[f"{prefix}.{local}"] = spec
        return out

    def aliases(self) -> dict[str, str]:
        """Names the file may store although the model takes them from another tensor."""
        n = self.spec.names
        return {f"{n['head']}.weight": f"{n['embedding']}.weight"} if self.tied_head else {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        for prefix, part in self._named_parts():
            own = {k[len(prefix) + 1:]: v for k, v in tensors.items() if k.startswith(prefix + ".")}
            if part is self.head and self.tied_head:
                own = {"weight": tensors[f"{self.spec.names['embedding']}.weight"]}
            if own or part.weight_specs():
                part.bind(own)

    # -- cache --------------------------------------------------------------
    def cache_needs(self):
        """For each cache entry of the schedule, the need of the layer that writes it."""
        needs = [None] * self.spec.cache_entries
        for run in self.spec.schedule:
            if run.writes_cache:
                needs[run.cache] = self.blocks[run.layer].cache_need()
        return needs


def expected_weights(spec: ModelSpec) -> dict[str, WeightSpec]:
    """Names, shapes and roles of the tensors a model of ``spec`` reads, without a device."""
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32, page_size=16,
                 max_positions=2, err=torch.zeros(2, dtype=torch.int32))
    return Model(spec, rt).weight_specs()
