"""The generalized delta rule as a mixer: a recurrent layer whose cache is one
``head_dim x head_dim`` float32 matrix per head and request, in a state slot of
the cache manager.

Per token and head (D = head_dim), with x the mixer's input:

    r, k, v, g, a_pre = five projections of x          (one product over the row-concatenated weights,
    t                 = tanh(w1 x)                       which also carries w1)
    w = exp(-decay_rate * sigmoid(w2 t + w0))          decay per key channel, in (exp(-decay_rate), 1)
    a = sigmoid(a_pre + a_bias)                        removal rate per key channel
    u = k / sqrt(sum(k^2) + key_eps)                   unit key
    S <- diag(w) S - (a * u) (u^T S) + k v^T           both terms read the old state
    o  = S^T r

then ``o`` is divided by its root mean square over the head, multiplied by a gain
over all heads and by ``sigmoid(g)``, and projected back by ``o_proj``.  The
projections are products in the activation type; ``w2 t`` leaves its product in
float32, and everything from there to the gated output is float32 inside one
kernel (``csrc/delta_rule.cu``), which runs a step's tokens of every request in
order from the state the step before left: a whole prompt, a portion and a
single decoded token take the same path.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache.manager import CacheRequirement
from ..weights.loader import ExpectedTensor
from .linear import Linear
from .registry import register_mixer


@register_mixer("general_delta")
class GeneralDeltaMixer:
    graph_safe = True          # request bounds and state slots are read on the device

    @staticmethod
    def expected_tensors(spec):
        width = spec.n_heads * spec.head_dim
        out = {}
        for name in (spec.r_proj, spec.k_proj, spec.v_proj, spec.g_proj, spec.a_proj):
            out[name] = ExpectedTensor((width, spec.hidden))
        out[spec.a_bias] = ExpectedTensor((width,))
        out[spec.w1] = ExpectedTensor((spec.decay_rank, spec.hidden))
        out[spec.w2] = ExpectedTensor((width, spec.decay_rank))
        out[spec.w0] = ExpectedTensor((width,))
        out[spec.out_gain] = ExpectedTensor((width,), init="gain")
        out[spec.o_proj] = ExpectedTensor((spec.hidden, width))
        return out

    def __init__(self, spec, tensors, rt):
        if not 1 <= spec.head_dim <= kernels.DELTA_RULE_MAX_DIM:
            raise ValueError(f"the delta-rule kernel takes head sizes up to {kernels.DELTA_RULE_MAX_DIM}, not {spec.head_dim}")
        self.spec = spec
        self.rt = rt
        self.width = spec.n_heads * spec.head_dim
        ws = [tensors[n] for n in (spec.r_proj, spec.k_proj, spec.v_proj, spec.g_proj, spec.a_proj, spec.w1)]
        dtype = torch.float32 if any(w.dtype is torch.float32 for w in ws) else ws[0].dtype
        self.proj = Linear(torch.cat([w.to(dtype) for w in ws], dim=0).contiguous(), rt, "delta_proj")
        self.w2 = Linear(tensors[spec.w2], rt, "delta_w2")
        self.o = Linear(tensors[spec.o_proj], rt, "o")
        vecs = [tensors[spec.a_bias], tensors[spec.w0], tensors[spec.out_gain]]
        vdtype = torch.float32 if any(v.dtype is torch.float32 for v in vecs) else vecs[0].dtype
        self.a_bias, self.w0, self.out_gain = (v.to(vdtype).contiguous() for v in vecs)

    def cache_requirement(self) -> CacheRequirement:
        s = self.spec
        return CacheRequirement(kind="state", state_shape=(s.n_heads, s.head_dim, s.head_dim),
                                state_dtype=torch.float32)

    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        s, rt, W = self.spec, self.rt, self.width
        n = x.shape[0]
        proj = self.proj(x, rt.ws.take("delta_proj", (n, 5 * W + s.decay_rank), rt.act_dtype))
        t = rt.ws.take("delta_lora", (n, s.decay_rank), rt.act_dtype)
        kernels.tanh(proj[:, 5 * W:], t)
        w_pre = self.w2(t, rt.ws.take("delta_w_pre", (n, W), torch.float32))
        r, k, v, g, a_pre = (proj[:, i * W:(i + 1) * W] for i in range(5))
        mixed = rt.ws.take("delta_mixed", (n, W), rt.act_dtype)
        kernels.delta_rule(r, k, v, a_pre, g, w_pre, self.a_bias, self.w0, self.out_gain, cache.state, mixed,
                           ctx.q_start, ctx.slots, ctx.n_requests, s.n_heads, s.head_dim, s.decay_rate, s.key_eps,
                           s.norm_eps, write_state=cache.write)
        return self.o(mixed, rt.ws.take("mixer_out", (n, s.hidden), rt.act_dtype))
