"""Convenience layer over ``Pipeline``/``Session`` that plays the role of the reference's test-side
client (utilities/pipeline.cpp:297-314, 388-497): it registers a graph's resources and constants,
creates the pipeline from SPIR-V assembly text, creates a session, allocates and binds device
memory (through torch, which is only used as an allocator and stream provider) and dispatches.
"""
from __future__ import annotations

import numpy as np
import torch

from . import NP_TO_DTYPE, Pipeline, Session
from .graph_builder import GraphBuilder


def make_pipeline(graph: GraphBuilder, flags: int = 0):
    """Registers the graph's resources and constants and lowers its SPIR-V assembly; needs no device.
    Returns ``(pipeline, input_keys, output_keys)`` with keys ``(set, binding, value)``."""
    pipeline = Pipeline(flags)
    in_keys, out_keys = [], []
    for v in graph.inputs:
        s, b = v.binding
        pipeline.bind_external(s, b, NP_TO_DTYPE[v.dtype], v.shape)
        in_keys.append((s, b, v))
    for v, s, b in graph.outputs:
        pipeline.bind_external(s, b, NP_TO_DTYPE[v.dtype], v.shape)
        out_keys.append((s, b, v))
    for cid, data in graph.constants.items():
        pipeline.add_constant(cid, data)
    pipeline.lower_spvasm(graph.spvasm())
    return pipeline, in_keys, out_keys


class GraphRunner:
    def __init__(self, graph: GraphBuilder, flags: int = 0, device: str | torch.device = "cuda"):
        self.graph = graph
        self.device = torch.device(device)
        self.pipeline, self._in_keys, self._out_keys = make_pipeline(graph, flags)
        self.session = Session(self.pipeline)
        size, align = self.session.memory_requirements()
        self.memory_size = size
        # torch's caching allocator hands out 512-byte aligned blocks
        self._arena = torch.empty(max(size, 1), dtype=torch.uint8, device=self.device)
        assert self._arena.data_ptr() % align == 0
        self.session.bind_memory(self._arena.data_ptr())
        self.inputs = [torch.empty(int(np.prod(v.shape)) * v.dtype.itemsize, dtype=torch.uint8, device=self.device)
                       for _, _, v in self._in_keys]
        self.outputs = [torch.zeros(int(np.prod(v.shape)) * v.dtype.itemsize, dtype=torch.uint8, device=self.device)
                        for _, _, v in self._out_keys]
        for (s, b, _), t in zip(self._in_keys, self.inputs):
            self.session.set_external(s, b, t.data_ptr())
        for (s, b, _), t in zip(self._out_keys, self.outputs):
            self.session.set_external(s, b, t.data_ptr())

    def set_inputs(self, arrays) -> None:
        for (_, _, v), t, a in zip(self._in_keys, self.inputs, arrays):
            a = np.ascontiguousarray(a, dtype=v.dtype).reshape(-1).view(np.uint8)
            t.copy_(torch.from_numpy(a))

    def dispatch(self, use_cuda_graph: bool = False) -> None:
        stream = torch.cuda.current_stream(self.device).cuda_stream
        if use_cuda_graph:
            self.session.dispatch_graph(stream)
        else:
            self.session.dispatch(stream)

    def get_outputs(self):
        torch.cuda.synchronize(self.device)
        return [t.cpu().numpy().view(v.dtype).reshape(v.shape) for (_, _, v), t in zip(self._out_keys, self.outputs)]

    def run(self, arrays, use_cuda_graph: bool = False):
        self.set_inputs(arrays)
        self.dispatch(use_cuda_graph)
        return self.get_outputs()
