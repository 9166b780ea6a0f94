"""The gated delta rule as a mixer: a recurrent layer whose cache is one ``head_dim x v_head_dim`` float32 matrix
per head and request, beside the last inputs of its short convolutions.

With x the mixer's input, per token:

    q, k (kv_heads x head_dim), v (heads x v_head_dim), b, a (heads), gate (heads x v_head_dim)
                       = six projections of x            (one product over the row-concatenated weights)
    q, k, v           <- silu(causal convolution over time, a filter per channel)
    q, k              <- unit vectors per head; q also times head_dim^-1/2
    beta = sigmoid(b),  g = exp(-exp(A_log) * softplus(a + dt_bias))        one number a head each
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q              per head; head h reads q/k head h // rep

then ``o`` is divided by its root mean square over the head, multiplied by a gain of the head's size and by
``silu(gate)``, and projected back by ``o_proj``.  The projections and the convolutions are in the activation
type; everything from there to the gated output is float32 inside one kernel (``csrc/gated_delta.cu``), which runs
a step's tokens of every request in order from the state the step before left: a whole prompt, a portion and a
single decoded token take the same path.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheRequirement
from ..weights.loader import ExpectedTensor
from .linear import Linear
from .registry import register_mixer


def conv_state_requirement(taps: int, channels: int, dtype: torch.dtype) -> CacheRequirement:
    """The state of a short convolution: a sequence's last ``taps - 1`` inputs, oldest first."""
    return CacheRequirement(kind="state", state_shape=(max(taps - 1, 0), channels), state_dtype=dtype)


def same_dtype(tensors: list[torch.Tensor]) -> list[torch.Tensor]:
    """Small tensors that one kernel reads with one type: float32 if any of them is, else as stored."""
    dtype = torch.float32 if any(t.dtype is torch.float32 for t in tensors) else tensors[0].dtype
    return [t.to(dtype).contiguous() for t in tensors]


@register_mixer("gated_delta")
class GatedDeltaMixer:
    graph_safe = True          # request bounds and state slots are read on the device

    @staticmethod
    def expected_tensors(spec):
        qk, vw = spec.n_kv_heads * spec.head_dim, spec.n_heads * spec.v_head_dim
        out = {}
        for name, conv, width in ((spec.q_proj, spec.q_conv, qk), (spec.k_proj, spec.k_conv, qk), (spec.v_proj, spec.v_conv, vw)):
            out[name] = ExpectedTensor((width, spec.hidden))
            out[conv.weight] = ExpectedTensor((width, conv.taps))
        out[spec.beta_proj] = ExpectedTensor((spec.n_heads, spec.hidden))
        out[spec.decay_log] = ExpectedTensor((spec.n_heads,))
        out[spec.out_gain] = ExpectedTensor((spec.v_head_dim,), init="gain")
        out[spec.decay_proj] = ExpectedTensor((spec.n_heads, spec.hidden))
        out[spec.decay_bias] = ExpectedTensor((spec.n_heads,))
        out[spec.gate_proj] = ExpectedTensor((vw, spec.hidden))
        out[spec.o_proj] = ExpectedTensor((spec.hidden, vw))
        return out

    def __init__(self, spec, tensors, rt):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError(f"{spec.n_heads} heads are not a multiple of {spec.n_kv_heads} q/k heads")
        taps = spec.q_conv.taps
        if not (spec.k_conv.taps == spec.v_conv.taps == taps and 1 <= taps <= kernels.CONV_MAX_TAPS):
            raise ValueError(f"the convolutions of q, k and v share one length of at most {kernels.CONV_MAX_TAPS} taps")
        if any(c.bias is not None for c in (spec.q_conv, spec.k_conv, spec.v_conv)):
            raise ValueError("the convolutions of the gated delta rule carry no bias")
        self.spec = spec
        self.rt = rt
        self.taps = taps
        self.qk = spec.n_kv_heads * spec.head_dim
        self.vw = spec.n_heads * spec.v_head_dim
        self.conv_width = 2 * self.qk + self.vw
        # columns of the one projection: q | k | v | gate | b | a  (the convolution runs over the first three)
        ws = [tensors[n] for n in (spec.q_proj, spec.k_proj, spec.v_proj, spec.gate_proj, spec.beta_proj, spec.decay_proj)]
        dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0).contiguous(), rt, "gated_delta_proj")
        self.proj_width = self.conv_width + self.vw + 2 * spec.n_heads
        convs = [tensors[c.weight] for c in (spec.q_conv, spec.k_conv, spec.v_conv)]
        cdtype = torch.float32 if any(c.dtype is torch.float32 for c in convs) else convs[0].dtype
        self.conv_weight = torch.cat([c.to(cdtype) for c in convs], dim=0).contiguous()
        self.a_log, self.dt_bias, self.out_gain = same_dtype([tensors[spec.decay_log], tensors[spec.decay_bias],
                                                             tensors[spec.out_gain]])
        self.o = Linear(tensors[spec.o_proj], rt, "o")
        kernels.gated_delta_library(spec.head_dim, spec.v_head_dim)      # built when the model is, not in its first step

    def cache_requirement(self) -> CacheRequirement:
        s = self.spec
        return CacheRequirement(kind="several", parts=(
            CacheRequirement(kind="state", state_shape=(s.n_heads, s.head_dim, s.v_head_dim), state_dtype=torch.float32),
            conv_state_requirement(self.taps, self.conv_width, self.rt.act_dtype)))

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        s, rt = self.spec, self.rt
        n = x.shape[0]
        state, conv_state = cache.parts
        proj = self.proj(x, rt.ws.take("gated_delta_proj", (n, self.proj_width), rt.act_dtype))
        conv = rt.ws.take("gated_delta_conv", (n, self.conv_width), rt.act_dtype)
        kernels.causal_conv(proj[:, :self.conv_width], self.conv_weight, None, conv_state.state, conv, ctx.q_start,
                            ctx.slots, ctx.n_requests, activation="silu", write_state=cache.write, max_q_len=ctx.max_q_len)
        c0 = self.conv_width
        gate = proj[:, c0:c0 + self.vw]
        b_pre = proj[:, c0 + self.vw:c0 + self.vw + s.n_heads]
        a_pre = proj[:, c0 + self.vw + s.n_heads:]
        mixed = rt.ws.take("gated_delta_mixed", (n, self.vw), rt.act_dtype)
        kernels.gated_delta(conv[:, :self.qk], conv[:, self.qk:2 * self.qk], conv[:, 2 * self.qk:], b_pre, a_pre, gate,
                            self.a_log, self.dt_bias, self.out_gain, state.state, mixed, ctx.q_start, ctx.slots,
                            ctx.n_requests, s.n_heads, s.n_kv_heads, s.head_dim, s.v_head_dim, s.key_eps, s.norm_eps,
                            write_state=cache.write)
        return self.o(mixed, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))
