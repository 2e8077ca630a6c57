"""Fixed-shape decode loop of `fused_recurrent_gated_delta_rule` replayed from a CUDA graph.

One decode step of the reference (`fla/ops/gated_delta_rule/fused_recurrent.py:210`, T = 1) is a single kernel of
about a tenth of a millisecond at 256 sequences x 16 heads; called through the functional API once per token, the
Python and launch overhead per call is of the same order. The decoder keeps the state (`[B, H, K, V]` fp32) and the
token vectors in fixed device buffers, captures the step once and replays it: the state is updated in place (every
(sequence, head) tile is read in full before the same CTA writes it back), nothing is allocated per step.

    dec = GatedDeltaRuleDecoder(B, H, K, V, dtype=torch.bfloat16, initial_state=h0)
    for t in range(steps):
        o = dec.step(q_t, k_t, v_t, g_t, beta_t)      # [B, 1, H, V], valid until the next step
    ht = dec.state                                     # [B, H, K, V] fp32
"""
from typing import Optional

import torch

from . import _lib
from .utils import Geometry


class GatedDeltaRuleDecoder:

    def __init__(self, batch: int, heads: int, head_k: int, head_v: int, dtype: torch.dtype = torch.bfloat16,
                 device: Optional[torch.device] = None, scale: Optional[float] = None,
                 initial_state: Optional[torch.Tensor] = None, use_graph: bool = True):
        if not torch.cuda.is_available():
            raise RuntimeError("GatedDeltaRuleDecoder needs a CUDA device (there is no CPU path)")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.scale = head_k ** -0.5 if scale is None else float(scale)
        assert self.scale > 0, "scale must be positive"
        B, H, K, V = batch, heads, head_k, head_v
        self.q = torch.zeros(B, 1, H, K, dtype=dtype, device=dev)
        self.k = torch.zeros(B, 1, H, K, dtype=dtype, device=dev)
        self.v = torch.zeros(B, 1, H, V, dtype=dtype, device=dev)
        self.g = torch.zeros(B, 1, H, dtype=torch.float32, device=dev)
        self.beta = torch.ones(B, 1, H, dtype=dtype, device=dev)
        self.o = torch.empty(B, 1, H, V, dtype=dtype, device=dev)
        self.state = torch.zeros(B, H, K, V, dtype=torch.float32, device=dev)
        if initial_state is not None:
            if tuple(initial_state.shape) != (B, H, K, V):
                raise ValueError(f"initial_state must have shape {(B, H, K, V)}, got {tuple(initial_state.shape)}")
            self.state.copy_(initial_state)
        self._geo = Geometry(self.k, self.v, None, False)
        self._graph = None
        self._graphs, self._steps = None, 0
        if use_graph:
            # capture on a side stream; the launch itself neither allocates nor synchronises
            keep = self.state.clone()
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream(dev))
            with torch.cuda.stream(side):
                self._launch()  # warm-up outside capture (module load, attribute setting)
            torch.cuda.current_stream(dev).wait_stream(side)
            self.state.copy_(keep)
            # two captures of the same step, one per direction of the walk over the state tiles: replays alternate, so a step
            # starts on the tiles its predecessor wrote last (still in L2)
            graphs = []
            for descending in (False, True):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._launch(descending)
                graphs.append(graph)
            self._graph, self._graphs = graphs[0], graphs
            self.state.copy_(keep)  # capture does not run the kernel, but keep the contract obvious

    def _launch(self, descending: bool = False):
        flags = _lib.F_INPLACE_STATE | (_lib.F_DESCENDING if descending else 0)
        _lib.call("flab_recurrent_delta_fwd", self.q, **self._geo.kw(), scale=self.scale, flags=flags, q=self.q, k=self.k,
                  v=self.v, beta=self.beta, g=self.g, h0=self.state, o=self.o, u=None, ht=self.state)

    def _run(self):
        self._steps += 1
        if self._graphs is not None:
            self._graphs[self._steps & 1].replay()
        else:
            self._launch(bool(self._steps & 1))

    @torch.no_grad()
    def step(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: Optional[torch.Tensor] = None,
             beta: Optional[torch.Tensor] = None) -> torch.Tensor:
        """One token per sequence: q, k `[B, 1, H, K]`, v `[B, 1, H, V]`, g (log space) and beta `[B, 1, H]`.
        Returns o `[B, 1, H, V]` (the decoder's own buffer: copy it if it must outlive the next step)."""
        self.q.copy_(q.view_as(self.q))
        self.k.copy_(k.view_as(self.k))
        self.v.copy_(v.view_as(self.v))
        # an omitted gate / beta means "none" for THIS step (g = 0: no decay, beta = 1), never the previous step's values
        if g is not None:
            self.g.copy_(g.view_as(self.g))
        else:
            self.g.zero_()
        if beta is not None:
            self.beta.copy_(beta.view_as(self.beta))
        else:
            self.beta.fill_(1)
        self._run()
        return self.o

    @torch.no_grad()
    def replay(self) -> torch.Tensor:
        """Run the step on whatever the input buffers (`.q .k .v .g .beta`) hold: for callers that write them in place."""
        self._run()
        return self.o
