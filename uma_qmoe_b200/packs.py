"""Pack objects the backends read experts from.

The backends only use the reader protocol of the reference's
``ExpertPackReader`` (``src/uma_qmoe/expert_pack.py:317-556``) and
``TargetPackReader`` (``src/uma_qmoe/target_pack.py:493-812``):

* ``mapping_count == 1``;
* ``tensor_views(name) -> (data memoryview, scales memoryview, metadata)`` with
  ``metadata["shape"]`` (and ``metadata["encoding"]`` for a TargetPack);
* ExpertPack: ``header["quantization"]["group_size"]``;
* TargetPack: ``layer_encoding(layer_index)``.

so the reference's own readers can be registered unchanged.  ``InMemoryPack``
implements the same protocol over host buffers, for synthetic weights (tests,
benchmarks) where no pack file exists.
"""

from __future__ import annotations

from typing import Any, Mapping

import numpy as np

from .formats import ENCODINGS, ContractError, PackedTensor, encode


def expert_tensor_name(layer: int, expert: int, projection: str) -> str:
    """Canonical tensor name inside a pack (``expert_pack.py:40-56`` in the reference)."""
    return f"model.layers.{layer}.mlp.experts.{expert}.{projection}.weight"


class InMemoryPack:
    """Host-resident pack with the TargetPack reader protocol (mixed encodings per layer)."""

    mapping_count = 1

    def __init__(self, layer_encodings: Mapping[int, str], model_id: str = "synthetic") -> None:
        for enc in layer_encodings.values():
            if enc not in ENCODINGS:
                raise ContractError(f"unsupported encoding {enc!r}")
        self._layer_encodings = dict(layer_encodings)
        self._tensors: dict[str, PackedTensor] = {}
        self.header = {"model": {"model_id": model_id},
                       "policy": {"layer_encodings": {str(k): v for k, v in layer_encodings.items()}},
                       "quantization": {"group_size": 128}}

    def layer_encoding(self, layer_index: int) -> str:
        try:
            return self._layer_encodings[layer_index]
        except KeyError as exc:
            raise ContractError(f"pack has no layer {layer_index}") from exc

    def add(self, name: str, values: Any, layer_index: int) -> None:
        """Quantise / encode one float tensor with its layer's encoding."""
        self.add_packed(name, encode(np.asarray(values), self.layer_encoding(layer_index)))

    def add_packed(self, name: str, tensor: PackedTensor) -> None:
        if name in self._tensors:
            raise ContractError(f"duplicate tensor name {name!r}")
        self._tensors[name] = tensor

    def tensor_views(self, name: str) -> tuple[memoryview, memoryview, Mapping[str, Any]]:
        try:
            t = self._tensors[name]
        except KeyError as exc:
            raise ContractError(f"pack has no tensor {name!r}") from exc
        meta = {"name": name, "shape": list(t.shape), "encoding": t.encoding,
                "group_size": None if t.encoding == "bf16_le" else 128}
        return memoryview(t.data), memoryview(t.scales), meta

    def names(self) -> list[str]:
        return list(self._tensors)

    def close(self) -> None:
        self._tensors.clear()
