"""Connections: how a sublayer reads the residual and how its output goes back into it.

Interface of a connection:

    tensor_specs() / bind(tensors)
    read                       # float32 [streams] or None: the coefficients a norm reads the streams with
    update(y) -> pending       # what the sublayer's output y becomes on its way into the residual

The residual of a token is `streams` 32-bit copies side by side in one row.  A block hands `read` to its norm
(`StreamRMSNorm.forward(..., read=...)`) and passes what `update` returns on as the pending delta; the norm that
reads the residual next applies it (parts/block.py::StreamMixedBlock).
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.registry import register_connection
from liteinfer_b200.parts.spec import TensorSpec


def _read_init(shape, generator):
    return 1.0 / shape[0] + 0.3 * torch.randn(shape, generator=generator)


def _write_init(shape, generator):
    return 1.0 + 0.3 * torch.randn(shape, generator=generator)


def _mix_init(shape, generator):
    return torch.eye(shape[0]) + 0.2 * torch.randn(shape, generator=generator)


def _gain_init(shape, generator):
    return 0.5 + torch.rand(shape, generator=generator)


class StreamConnection:
    """Residual streams with learned read, write and mixing coefficients, and a gain per channel on the sublayer's
    output: u = sum_s in[s] x_s is what the sublayer sees (after its norm); afterwards, all streams at once from
    the old ones, x_t <- sum_s mix[s, t] x_s + out[t] * gain * y.  Tensors: `in` [S], `out` [S], `mix` [S, S]
    (indexed [from, to]) and `gain` [width], all kept 32-bit.  `learned` False: one stream and the plain sum
    x <- x + gain * y, with no coefficient tensors; `gain` False: no gain tensor."""

    def __init__(self, streams: int, width: int, dtype: torch.dtype, device: torch.device, learned: bool = True,
                 gain: bool = True) -> None:
        if streams < 1:
            raise ValueError("a residual has at least one stream")
        if not learned and streams != 1:
            raise ValueError("several streams need their coefficients (learned=True)")
        self.streams, self.width, self.learned, self.has_gain = streams, width, learned, gain
        self.device = device
        self.read: torch.Tensor | None = None
        self.write = self.mix = self.gain = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        s = self.streams
        specs: dict[str, TensorSpec] = {}
        if self.learned:
            specs.update({"in": TensorSpec((s,), kind="f32", init=_read_init),
                          "out": TensorSpec((s,), kind="f32", init=_write_init),
                          "mix": TensorSpec((s, s), kind="f32", init=_mix_init)})
        if self.has_gain:
            specs["gain"] = TensorSpec((self.width,), kind="f32", init=_gain_init)
        return specs

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        if self.learned:
            self.read, self.write, self.mix = (tensors[n].contiguous() for n in ("in", "out", "mix"))
        else:
            self.read = None
            self.write = torch.ones(1, dtype=torch.float32, device=self.device)
            self.mix = torch.ones((1, 1), dtype=torch.float32, device=self.device)
        self.gain = tensors["gain"].contiguous() if self.has_gain else None

    def update(self, y: torch.Tensor) -> "ops.StreamUpdate":
        return ops.StreamUpdate(y, self.gain, self.write, self.mix)


register_connection("stream_mix", StreamConnection)
