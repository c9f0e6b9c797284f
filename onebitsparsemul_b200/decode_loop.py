"""A Llama-shaped stack of linear layers and a CUDA-graph decode loop over it.

The reference's model-replace demo (tests/python/test_model_replace.py:22-44) walks a TinyLlama checkpoint and
swaps every ``nn.Linear`` for a ``BinaryLinear_2_4``. The checkpoint is not part of that repository; what the
flow exercises is the set of linear layers of a decoder block -- q/k/v/o (hidden x hidden), gate/up
(intermediate x hidden), down (hidden x intermediate) -- called one token at a time. `LlamaShapedStack` is
exactly that set with random weights; the attention and normalisation arithmetic between the layers, which the
one-bit path does not touch, is replaced by cheap element-wise glue with the same data flow, so that every
linear layer reads the output of an earlier one.

`GraphedDecoder` captures one step of the (replaced) stack in a CUDA graph and replays it per token: the
few-token kernels then run back to back without host launches between them, each grid starting while its
predecessor drains (programmatic dependent launch). This is the measurement of the decode regime as a model
sees it: a single call moves 3-9 MB and costs less at HBM speed than a kernel launch.
"""
from __future__ import annotations

import torch
import torch.nn as nn
import torch.nn.functional as F


class LlamaShapedBlock(nn.Module):
    """The seven linear layers of a Llama-style decoder block (no biases, like the original).

    With ``fused=True`` the three projections that read the same input are one layer (``qkv_proj``, 3 * hidden rows) and
    so are gate and up (``gate_up_proj``, 2 * intermediate rows), as serving stacks lay them out: four GEMMs per
    block instead of seven, each with more row blocks to spread over the SMs. The arithmetic is the same."""

    def __init__(self, hidden: int = 4096, intermediate: int = 11008, dtype=torch.float16, device=None, fused: bool = False):
        super().__init__()
        kw = dict(bias=False, dtype=dtype, device=device)
        self.fused, self.hidden, self.intermediate = fused, hidden, intermediate
        if fused:
            self.qkv_proj = nn.Linear(hidden, 3 * hidden, **kw)
            self.gate_up_proj = nn.Linear(hidden, 2 * intermediate, **kw)
        else:
            self.q_proj, self.k_proj = nn.Linear(hidden, hidden, **kw), nn.Linear(hidden, hidden, **kw)
            self.v_proj = nn.Linear(hidden, hidden, **kw)
            self.gate_proj, self.up_proj = nn.Linear(hidden, intermediate, **kw), nn.Linear(hidden, intermediate, **kw)
        self.o_proj = nn.Linear(hidden, hidden, **kw)
        self.down_proj = nn.Linear(intermediate, hidden, **kw)

    def forward(self, x):
        """x: (tokens, hidden). Element-wise glue stands in for attention and normalisation."""
        if self.fused:
            q, k, v = self.qkv_proj(x).split(self.hidden, dim=-1)
        else:
            q, k, v = self.q_proj(x), self.k_proj(x), self.v_proj(x)
        h = x + self.o_proj(torch.tanh(q) * torch.sigmoid(k) + 0.5 * v)
        h = h * torch.rsqrt(h.float().pow(2).mean(-1, keepdim=True) + 1e-5).to(h.dtype)
        if self.fused:
            gate, up = self.gate_up_proj(h).split(self.intermediate, dim=-1)
        else:
            gate, up = self.gate_proj(h), self.up_proj(h)
        return h + self.down_proj(F.silu(gate) * up)


class LlamaShapedStack(nn.Module):
    def __init__(self, blocks: int = 4, hidden: int = 4096, intermediate: int = 11008, dtype=torch.float16, device=None, seed: int = 0,
                 fused: bool = False):
        super().__init__()
        self.hidden, self.intermediate = hidden, intermediate
        self.blocks = nn.ModuleList([LlamaShapedBlock(hidden, intermediate, dtype, device, fused) for _ in range(blocks)])
        g = torch.Generator(device="cpu")
        g.manual_seed(seed)
        with torch.no_grad():
            for p in self.parameters():                          # N(0, 1 / fan_in): activations keep their scale
                p.copy_((torch.randn(p.shape, generator=g) / p.shape[1] ** 0.5).to(p.dtype))

    def forward(self, x):
        for b in self.blocks:
            x = b(x)
        return x

    def linear_layers(self):
        return [m for m in self.modules() if isinstance(m, nn.Linear) or type(m).__name__ == "BinaryLinear_2_4"]


class GraphedDecoder:
    """One decode step of `model` for a fixed number of tokens, captured in a CUDA graph.

    The first calls run eagerly (they make the library allocate its per-device status word and mark the packed
    weights as long-lived); the capture follows. `step(x)` copies x into the graph's input, replays, and returns
    the graph's output tensor (overwritten by the next step)."""

    def __init__(self, model: nn.Module, tokens: int, hidden: int, device="cuda", warmup: int = 3):
        self.model = model
        self.x = torch.zeros((tokens, hidden), dtype=torch.float16, device=device)
        side = torch.cuda.Stream(device=device)
        side.wait_stream(torch.cuda.current_stream(device))
        with torch.cuda.stream(side), torch.no_grad():
            for _ in range(warmup):
                self.model(self.x)
        torch.cuda.current_stream(device).wait_stream(side)
        torch.cuda.synchronize(device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph), torch.no_grad():
            self.y = self.model(self.x)

    def step(self, x):
        self.x.copy_(x)
        self.graph.replay()
        return self.y


def measure_decode(model: nn.Module, hidden: int, tokens: int = 1, steps: int = 50, device="cuda"):
    """Device time of one decode step through the graph, per token step and per linear layer."""
    dec = GraphedDecoder(model, tokens, hidden, device)
    x = torch.randn((tokens, hidden), device=device, dtype=torch.float32).to(torch.float16)
    for _ in range(3):
        dec.step(x)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        dec.graph.replay()
    e1.record()
    torch.cuda.synchronize(device)
    us = e0.elapsed_time(e1) * 1e3 / steps
    layers = [m for m in model.modules() if type(m).__name__ == "BinaryLinear_2_4"]
    packed_bytes = sum(m.bits_tile.numel() + m.meta_tile.numel() for m in layers)
    return {"tokens": tokens, "linear_layers": len(layers), "us_per_step": us, "us_per_linear_layer": us / max(1, len(layers)),
            "steps_per_s": 1e6 / us, "tokens_per_s": tokens * 1e6 / us, "packed_weight_bytes": packed_bytes,
            "weight_gbs": packed_bytes / us / 1e3}
