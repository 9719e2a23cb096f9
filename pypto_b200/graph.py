"""CUDA-graph capture of the operators: the serving-side mode the reference offers for its own
operators (graph-capture integration, docs/tutorials/network_integration/PyTorch集成和接入.md:5-6;
examples/03_advanced/aclgraph/aclgraph.py).

An operator call is capturable as it is: it allocates nothing once its workspace for the capturing
stream exists, never synchronises, and reads the sequence lengths on the device. `CapturedCall` does the
one warm-up call on the capture stream (which creates that workspace), records the call into a
`torch.cuda.CUDAGraph` and replays it; the tensors passed in are the graph's static inputs and outputs:
update them in place between replays.
"""
from __future__ import annotations

import torch

from . import ops


class CapturedCall:
    """One operator call recorded into a CUDA graph.

        step = CapturedCall(pypto_b200.decode_indexer_attention_quant, idx_query, ..., topk_res, attention_out)
        idx_query.copy_(new_queries); ...          # refresh the static inputs in place
        step.replay()                              # on the current stream
    """

    def __init__(self, op, *args, **kwargs):
        if not callable(op):
            raise TypeError("op must be one of the pypto_b200 operators")
        dev = None
        for a in args:
            t = getattr(a, "tensor", a)
            if isinstance(t, torch.Tensor) and t.is_cuda:
                dev = t.device
                break
        if dev is None:
            raise RuntimeError("no CUDA tensor among the arguments: there is nothing to capture")
        self.device = dev
        self._keep = (args, kwargs)  # the graph reads and writes these buffers: keep them alive
        self._stream = torch.cuda.Stream(dev)
        self._stream.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(self._stream):
            op(*args, **kwargs)  # warm-up: creates the workspace of this stream, outside the capture
        torch.cuda.current_stream(dev).wait_stream(self._stream)
        torch.cuda.synchronize(dev)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, stream=self._stream):
            op(*args, **kwargs)

    def replay(self):
        self.graph.replay()

    def workspace_status(self):
        """Device status words of the captured call's workspace (synchronises the capture stream)."""
        with torch.cuda.stream(self._stream):
            return ops.workspace_status(self.device)
