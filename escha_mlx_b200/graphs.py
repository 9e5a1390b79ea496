"""CUDA-graph replay of a fixed-shape call.

A batch-1 coded layer is a dozen kernels of a few microseconds each, so on B200
the Python and launch cost of issuing them one by one exceeds their run time.
The kernels are written to be capturable (no host synchronisation, no
allocation inside the C ABI, static shapes, split-K counters left zero on exit),
so a caller with a fixed batch shape captures its forward once and replays it.
The reference gets the same effect from MLX's lazy graph (escha_mlx/msl.py:11-12
"no host sync in the MoE path").
"""
from __future__ import annotations

from typing import Callable, Sequence

import torch


class GraphedCall:
    """Capture ``fn(*static_inputs)`` once; ``__call__`` copies new inputs into the
    static buffers and replays.  Outputs are the graph's static output tensors
    (valid until the next replay).

    ``fn`` must allocate its outputs through torch (the capture's private memory
    pool keeps them alive) and must only launch work on the current stream.
    """

    def __init__(self, fn: Callable, example_inputs: Sequence[torch.Tensor], warmup: int = 3,
                 stream: torch.cuda.Stream | None = None) -> None:
        self._inputs = [t.clone() for t in example_inputs]
        self._stream = stream or torch.cuda.Stream()
        self._graph = torch.cuda.CUDAGraph()
        self._stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self._stream):
            for _ in range(warmup):      # sizes workspaces and LUTs outside the capture
                fn(*self._inputs)
        self._stream.synchronize()
        with torch.cuda.graph(self._graph, stream=self._stream):
            self._outputs = fn(*self._inputs)
        torch.cuda.current_stream().wait_stream(self._stream)

    @property
    def inputs(self) -> list[torch.Tensor]:
        return self._inputs

    @property
    def outputs(self):
        return self._outputs

    def replay(self) -> None:
        self._graph.replay()

    def close(self) -> None:
        """Destroy the captured graph and drop its static tensors.  A graph that
        captured NCCL collectives keeps a reference on the communicator, and
        NCCL's communicator teardown waits until every such graph is gone: call
        this on each graphed call before ``destroy_process_group()``."""
        self._graph.reset()
        self._outputs = None
        self._inputs = []

    def __call__(self, *inputs: torch.Tensor):
        for dst, src in zip(self._inputs, inputs):
            dst.copy_(src, non_blocking=True)
        self._graph.replay()
        return self._outputs
