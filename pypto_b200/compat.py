"""Call-site compatibility with the reference's front end.

`from_torch` and `Tensor` mirror `pypto.from_torch` / `pypto.Tensor`
(python/pypto/converter.py:36-112, python/pypto/tensor.py:22-41): a handle that carries the data
pointer, shape, dtype and device of a contiguous torch tensor. `dynamic_axis`, `name` and
`tensor_format` are compile hints of the reference's tracing compiler and are ignored here.
`SaTileShapeConfig` (sparse_flash_attention_quant_impl.py:35-42) and `LightningIndexerConfigs`
(deepseekv32_lightning_indexer_quant.py:24-47) are Ascend tiling knobs: accepted so that call sites
stay source-compatible, never read.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch


class Tensor:
    """Handle to a contiguous torch tensor (what `pypto.from_torch` returns)."""

    __slots__ = ("_t", "name", "shape", "ori_shape", "dtype", "device", "data_ptr")

    def __init__(self, t: torch.Tensor, name: str = "", dyn_shape=None):
        self._t = t
        self.name = name
        self.ori_shape = list(t.shape)
        self.shape = list(dyn_shape) if dyn_shape is not None else list(t.shape)
        self.dtype = t.dtype
        self.device = t.device
        self.data_ptr = t.data_ptr()

    def torch(self) -> torch.Tensor:
        return self._t


def from_torch(tensor, name: str = "", dynamic_axis: Optional[List[int]] = None, tensor_format=None) -> Tensor:
    if not isinstance(tensor, torch.Tensor):
        raise TypeError("input type is not currently supported.")
    if not tensor.is_contiguous():
        raise RuntimeError("not all tensors are contiguous")
    if tensor.dim() == 0:
        return Tensor(tensor.reshape(1), name)
    dyn = list(tensor.shape)
    for axis in dynamic_axis or []:
        dyn[axis] = -1
    return Tensor(tensor, name, dyn)


def unwrap(x, what: str) -> torch.Tensor:
    """Accepts a `Tensor` handle or a raw torch tensor; enforces the reference's contiguity rule."""
    if isinstance(x, Tensor):
        return x.torch()
    if isinstance(x, torch.Tensor):
        if not x.is_contiguous():
            raise RuntimeError(f"not all tensors are contiguous ({what})")
        return x
    raise TypeError(f"{what}: input type is not currently supported.")


@dataclass
class SaTileShapeConfig:
    g_tile: int = 128
    s_kv_tile: int = 2048
    c1_tile_shape: list = field(default_factory=lambda: [128, 128, 128, 128, 128, 128])
    v1_tile_shape: list = field(default_factory=lambda: [8, 2048])
    c2_tile_shape: list = field(default_factory=lambda: [128, 128, 128, 128, 128, 128])
    v2_tile_shape: list = field(default_factory=lambda: [64, 128])


@dataclass
class LightningIndexerConfigs:
    mg_copy_in_upper_bound: int = 2 * 1024 * 1024
    pg_upper_bound: int = 16 * 8192
    cube_l1_reuse_setting: dict = field(default_factory=lambda: {0: 16})
    vec_merge_mode: int = 2
    vec_nbuffer_setting: dict = field(default_factory=lambda: {-1: 16})
    s1_tile: int = 2
    topk_tile: int = 16384
    c1_tile: list = field(default_factory=lambda: [64, 64, 128, 128, 128, 128])
    c2_tile: list = field(default_factory=lambda: [128, 128, 64, 64, 128, 128])
    # the 1/2048 scale and the ReLU are part of the operator's arithmetic, not options
    extend_param: dict = field(default_factory=lambda: {"scale": 1 / 2048.0, "relu_type": "RELU"})
