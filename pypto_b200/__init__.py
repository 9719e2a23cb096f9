"""B200-native (sm_100a) implementation of the quantized DeepSeek-V3.2 sparse-attention decode
path, behind the operator names of the reference's examples/models/deepseek_v32_exp package."""
import importlib

from .compat import LightningIndexerConfigs, SaTileShapeConfig, Tensor, from_torch  # noqa: F401

_OPS = (
    "lightning_indexer_decode", "lightning_indexer_scores", "lightning_indexer_topk",
    "lightning_indexer_topk_nonquant", "decode_indexer_attention",
    "sparse_flash_attention_quant_d", "sparse_flash_attention_quant_p",
    "sparse_attention_antiquant_d", "sparse_attention_antiquant_p",
    "mla_indexer_prolog_quant_d", "mla_indexer_prolog_quant_p", "pack_kv_cache",
    "mla_indexer_prolog", "decode_indexer_attention_layer",
    "decode_indexer_attention_quant", "workspace_status", "reset_workspace_status", "launch_count",
)


def __getattr__(name):
    if name == "CapturedCall":
        return importlib.import_module(".graph", __name__).CapturedCall
    # operators resolve lazily so that `pypto_b200.inputs` / `pypto_b200.build` import before the library is built
    if name in _OPS:
        return getattr(importlib.import_module(".ops", __name__), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
