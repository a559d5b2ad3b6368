"""How a sublayer reads and rejoins a residual stream that is kept as several copies (hyper-connections).

With ``streams`` copies x_1 .. x_s of the residual stream, a sublayer reads  u = sum_s read[s] x_s  and its result y
joins every copy at once,  x_t <- sum_s mix[s, t] x_s + write[t] y  (``mix`` is indexed [from, to]).

"learned": the three tensors ``in`` [s], ``out`` [s] and ``mix`` [s, s] come from the checkpoint.
"plain":   one stream, read = write = mix = 1: the ordinary residual addition x += y.

The coefficients are held in float32; the streams themselves are float32 (parts/block.py "hyper_prenorm",
csrc/streams.cu).  The reference has one residual stream (src/model/qwen.cpp:300-318).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import FAMILIES, ParamSpec, Part, _register

STREAM_MIXINGS: Dict[str, type] = {}
FAMILIES["stream_mixing"] = STREAM_MIXINGS


def register_stream_mixing(name):
    return _register(STREAM_MIXINGS, name)


class StreamMixing(Part):
    """``read`` [s], ``write`` [s] and ``mix`` [s, s] as float32 device tensors once loaded; ``streams`` their number."""
    streams: int = 1
    read: Optional[torch.Tensor] = None
    write: Optional[torch.Tensor] = None
    mix: Optional[torch.Tensor] = None

    def product_weights(self):
        return []


@register_stream_mixing("learned")
class LearnedStreamMixing(StreamMixing):
    def __init__(self, streams: int, dtype, device):
        if not 1 <= streams <= ops.STREAMS_MAX:
            raise ValueError(f"stream mixing: between 1 and {ops.STREAMS_MAX} streams, got {streams}")
        self.streams = int(streams)

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = self.streams
        # random weights: reading coefficients and write factors around 1, the mixing matrix around the identity
        return {"in": ParamSpec((s,), "gain"), "out": ParamSpec((s,), "gain"), "mix": ParamSpec((s, s), "identity")}

    def load_params(self, tensors):
        self.read = tensors["in"].to(torch.float32).contiguous()
        self.write = tensors["out"].to(torch.float32).contiguous()
        self.mix = tensors["mix"].to(torch.float32).contiguous()


@register_stream_mixing("plain")
class PlainStream(StreamMixing):
    def __init__(self, dtype, device):
        self.streams = 1
        self.device = device
        if torch.device(device).type != "meta":
            self.read = torch.ones(1, dtype=torch.float32, device=device)
            self.write = torch.ones(1, dtype=torch.float32, device=device)
            self.mix = torch.ones(1, 1, dtype=torch.float32, device=device)
