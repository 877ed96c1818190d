"""The gated delta-rule mixer: a linear recurrence over a matrix state per head, with short convolutions.

Per token, with h the mixer's input:

    q, k, v = silu(conv(W_q h)), silu(conv(W_k h)), silu(conv(W_v h))     # conv: causal, per channel, a few taps
    q, k    = q / |q| * dim^-0.5, k / |k|                                  # per head, |x| = sqrt(sum x^2 + 1e-6)
    beta    = sigmoid(W_b h);  g = exp(-exp(A_log) * softplus(W_a h + dt_bias))      # per head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q           # S [dim, vdim] per head, 32-bit
    y = W_o (norm_weight * o / rms(o) * silu(W_g h))                       # rms per head over vdim

q and k have `kv_heads` heads of `dim`; v, the gate and the state have `heads` heads (head i reads q/k head
i // (heads / kv_heads)).  What a request keeps between steps is its state S and the last taps - 1 inputs of
the convolutions: two `StateNeed`s, so a sequence may arrive whole, in portions or one token at a time.
Everything of the recurrence besides the projections and the convolutions is computed in 32-bit.
"""

from __future__ import annotations

import torch

from liteinfer_b200 import ops
from liteinfer_b200.parts.context import LayerCache, StateNeed, StepContext
from liteinfer_b200.parts.registry import register_mixer
from liteinfer_b200.parts.spec import TensorSpec


def _decay_init(shape, generator):
    """A_log such that exp(A_log) lies in [1, 8]."""
    return torch.log(1.0 + 7.0 * torch.rand(shape, generator=generator))


def _conv_init(shape, generator):
    return 0.4 * torch.randn(shape, generator=generator)


class GatedDeltaRule:
    def __init__(self, hidden_size: int, heads: int, kv_heads: int, dim: int, vdim: int, conv: int, norm_eps: float,
                 dtype: torch.dtype, device: torch.device, state_name: str = "delta", tail_name: str = "conv") -> None:
        if heads % kv_heads:
            raise ValueError(f"heads={heads} is not a multiple of kv_heads={kv_heads}")
        if conv < 1:
            raise ValueError("the convolutions need at least one tap")
        self.hidden_size, self.heads, self.kv_heads, self.dim, self.vdim = hidden_size, heads, kv_heads, dim, vdim
        self.taps, self.norm_eps = conv, float(norm_eps)
        self.state_name, self.tail_name = state_name, tail_name
        self.qk_width, self.v_width = kv_heads * dim, heads * vdim
        self.channels = 2 * self.qk_width + self.v_width             # what the convolutions run over: q, k, v
        self.in_weight = self.conv_weight = self.a_log = self.dt_bias = self.norm_weight = self.o_weight = None

    def tensor_specs(self) -> dict[str, TensorSpec]:
        d, qk, v, h = self.hidden_size, self.qk_width, self.v_width, self.heads
        return {
            "q_proj.weight": TensorSpec((qk, d)), "q_conv.weight": TensorSpec((qk, self.taps), init=_conv_init),
            "k_proj.weight": TensorSpec((qk, d)), "k_conv.weight": TensorSpec((qk, self.taps), init=_conv_init),
            "v_proj.weight": TensorSpec((v, d)), "v_conv.weight": TensorSpec((v, self.taps), init=_conv_init),
            "b_proj.weight": TensorSpec((h, d)), "a_proj.weight": TensorSpec((h, d)),
            "A_log": TensorSpec((h,), kind="f32", init=_decay_init), "dt_bias": TensorSpec((h,), kind="f32"),
            "g_proj.weight": TensorSpec((v, d)), "norm.weight": TensorSpec((self.vdim,), kind="f32", init="ones_normal"),
            "o_proj.weight": TensorSpec((d, v)),
        }

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        # One product for everything that reads h: [q | k | v | gate | beta | decay], padded to a multiple of 16 rows.
        parts = [tensors[n + "_proj.weight"] for n in ("q", "k", "v", "g", "b", "a")]
        rows = sum(p.shape[0] for p in parts)
        pad = -rows % 16
        if pad:
            parts.append(torch.zeros((pad, self.hidden_size), dtype=parts[0].dtype, device=parts[0].device))
        self.in_weight = torch.cat(parts).contiguous()
        # The taps of q, k and v's channels side by side, tap by tap: [taps, channels].
        self.conv_weight = torch.cat([tensors[n + "_conv.weight"] for n in ("q", "k", "v")]).t().contiguous()
        self.a_log, self.dt_bias = tensors["A_log"].contiguous(), tensors["dt_bias"].contiguous()
        self.norm_weight, self.o_weight = tensors["norm.weight"].contiguous(), tensors["o_proj.weight"]

    def cache_needs(self) -> tuple:
        return (StateNeed((self.heads, self.vdim, self.dim), "f32", name=self.state_name),     # S^T: column by column
                StateNeed((self.taps - 1, self.channels), "weight", name=self.tail_name))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: LayerCache) -> torch.Tensor:
        if cache.read_only:
            raise ValueError("a delta-rule mixer cannot read another stop's state: its state moves with every token")
        tokens = x.shape[0]
        state, tail = cache.states[self.state_name], cache.states[self.tail_name]
        proj = ops.linear(x, self.in_weight, None)
        c, v = self.channels, self.v_width
        conved = torch.empty((tokens, c), dtype=x.dtype, device=x.device)
        ops.short_conv_step(proj[:, :c], self.conv_weight, tail, ctx.seq_of_token, ctx.query_start_loc, ctx.state_slots,
                            ctx.num_seqs, conved, "silu", single_tokens=ctx.max_query_len == 1)
        read = torch.empty((tokens, v), dtype=torch.float32, device=x.device)
        ops.gated_delta_rule(conved, proj[:, c + v:c + v + 2 * self.heads], self.a_log, self.dt_bias, state,
                             ctx.query_start_loc, ctx.state_slots, ctx.num_seqs, self.heads, self.kv_heads, self.dim,
                             self.vdim, read, ctx.max_query_len)
        gated = torch.empty((tokens, v), dtype=x.dtype, device=x.device)
        ops.gated_rmsnorm(read, proj[:, c:c + v], self.norm_weight, self.norm_eps, gated, self.heads)
        return ops.linear(gated, self.o_weight, None)


register_mixer("gated_delta_rule", GatedDeltaRule)
