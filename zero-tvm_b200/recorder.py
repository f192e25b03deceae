"""A decode step as one CUDA graph: the engine records a fixed sequence of dispatches per token
(src/zero-tvm/engine-core.ts:2194-2202) and submits it as one command buffer; here the same sequence of calls through
the C ABI is captured once into a CUDA graph and replayed per token, so a step costs one launch on the host.

    rec = DecodeRecorder(backend)
    rec.dispatch("int4_matmul_sg_tiled_vec4h_affine", [qkv, x, s, W, pod, b], grid)   # any method of the backend
    rec.router_logits("moe_router_logits", [...], grid); rec.router_topk(...); ...
    step = rec.capture()        # one eager pass first (function attributes, work buffers), then the capture
    step.replay()               # every buffer is bound by address, as in the engine's bind groups

Only calls of this library are recorded; whatever else a step needs (attention, norms) would be captured by its own
owner on the same stream. torch is the owner of the stream and the graph object (plumbing).
"""
from __future__ import annotations

from typing import Callable, List, Tuple


class DecodeRecorder:
    def __init__(self, backend):
        self.be = backend
        self._calls: List[Tuple[Callable, tuple, dict]] = []
        self._graph = None
        self._stream = None

    # -- recording: the same surface as CudaMatmulBackend, minus the stream (the recorder owns it) --------------------
    def dispatch(self, entry, bindings, grid=(1, 1, 1)):
        self._calls.append((self.be.dispatch, (entry, list(bindings), tuple(grid)), {}))

    def router_logits(self, entry, bindings, grid=(1, 1, 1)):
        self._calls.append((self.be.dispatch_router_logits, (entry, list(bindings), tuple(grid)), {}))

    def embedding(self, entry, bindings, D):
        self._calls.append((self.be.dispatch_embedding, (entry, list(bindings), D), {}))

    def router_topk(self, ids, scores, logits, E, K, norm_topk, has_shared, tokens):
        self._calls.append((self.be.moe_router_topk, (ids, scores, logits, E, K, norm_topk, has_shared, tokens), {}))

    def silu_mul(self, out, gate_up, rows, ffn):
        self._calls.append((self.be.silu_mul, (out, gate_up, rows, ffn), {}))

    def moe_combine(self, out, y_slots, scores, tokens, slots, d):
        self._calls.append((self.be.moe_combine, (out, y_slots, scores, tokens, slots, d), {}))

    def __len__(self):
        return len(self._calls)

    def _run(self, stream):
        for fn, args, kw in self._calls:
            fn(*args, stream=stream, **kw)

    def run_eager(self, stream=None):
        """The recorded sequence as plain launches on `stream` (default: torch's current stream)."""
        import torch
        s = stream if stream is not None else torch.cuda.current_stream()
        self._run(s.cuda_stream if s.cuda_stream else 1)

    def capture(self, plan_reuse: bool = True):
        """One eager pass (sets kernel attributes, grows the context's work buffers: neither may happen inside a
        capture), then the capture. plan_reuse: the MoE matmuls of the step share one expert-sorted plan per id list
        (valid because, inside the recorded sequence, only the recorded router writes the id list)."""
        import torch
        if not self._calls:
            raise ValueError("nothing recorded")
        self._stream = torch.cuda.Stream()
        self._stream.wait_stream(torch.cuda.current_stream())
        self.be.ctx.moe_plan_reuse(plan_reuse)
        try:
            with torch.cuda.stream(self._stream):
                self._run(self._stream.cuda_stream)
                self._stream.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=self._stream):
                    self.be.ctx.moe_plan_reuse(plan_reuse)          # drops any plan: the captured step builds its own
                    self._run(self._stream.cuda_stream)
                self._stream.synchronize()
        finally:
            self.be.ctx.moe_plan_reuse(False)
        self._graph = g
        return self

    def replay(self):
        if self._graph is None:
            raise RuntimeError("capture() first")
        self._graph.replay()

    def synchronize(self):
        self._stream.synchronize()
