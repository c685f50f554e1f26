"""Routed feed-forward: many small experts of which every token uses a few, and optionally one
shared expert that every token uses.

    z = W_router h (fp32),  s = sigmoid(z) (or softmax over the experts)
    the ``top_k`` experts with the largest s are chosen; their weights are those s, as they are
        (or divided by their sum: ``renormalize``)
    expert(u) = W_down act(W_up u), act(z) = relu(z)^2, no biases
    y = sum_e expert_e(w_e h)                 the weight scales the expert's input (``weight_on="input"``)
        or sum_e w_e expert_e(h)              (``weight_on="output"``)
      + sigmoid(w_sg . h) * shared(h)         the shared expert, if any, with a gate of one number per token
                                              (``shared_gate``; without it the shared expert is added as it is)

Options that other designs use:
    ``activation="swiglu"``    expert(u) = W_down (silu(W_gate u) * W_up u)     (tensors ``e<i>.gate``, ``e<i>.up``, ``e<i>.down``)
    ``correction``             a vector (tensor ``correction``) added to the scores for the choice only; the weights
                               are the scores without it
    ``groups``, ``keep``       the experts form ``groups`` equal groups of neighbours; a group's mark is its largest
                               choice score (``group_mark="top2_sum"``: the sum of its two largest), and only
                               experts of the ``keep`` best groups can be chosen
    ``route_scale``            multiplies the weights
    ``identity``               the last ``identity`` of the router's num_experts + identity outputs are experts
                               without tensors whose output is their input (times the weight); they take part in
                               the scores, the groups and the choice like any other

The experts' matrices are kept stacked, [experts, ff, hidden] and [experts, hidden, ff], so that a
kernel reaches an expert by its index; the checkpoint has them one by one (``e<i>.up``, ``e<i>.down``).
"""
from __future__ import annotations

from typing import Dict

import torch

from ..registry import register_feed_forward
from .base import FeedForward, ParamSpec, StepContext


@register_feed_forward("none")
class NoFeedForward(FeedForward):
    """A layer without a feed-forward: the arrangement skips it and its norm."""
    is_identity = True

    def __init__(self, hidden_size: int):
        self.hidden = int(hidden_size)

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        return


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, num_experts: int, top_k: int, expert_ff: int, shared_ff: int = 0,
                 shared_gate: bool = True, score: str = "sigmoid", renormalize: bool = False,
                 weight_on: str = "input", activation: str = "relu2", correction: bool = False, groups: int = 1,
                 keep: int = 1, route_scale: float = 1.0, identity: int = 0, group_mark: str = "max"):
        self.hidden, self.E, self.top, self.F = int(hidden_size), int(num_experts), int(top_k), int(expert_ff)
        self.SF, self.shared_gate = int(shared_ff), bool(shared_gate) and int(shared_ff) > 0
        if not 0 < self.top <= self.E + int(identity):
            raise ValueError(f"routed experts: top_k={self.top} of {self.E} experts")
        if score not in ("sigmoid", "softmax") or weight_on not in ("input", "output"):
            raise ValueError(f"routed experts: score={score!r}, weight_on={weight_on!r}")
        self.score, self.renormalize, self.scale_input = score, bool(renormalize), weight_on == "input"
        if activation not in ("relu2", "swiglu"):
            raise ValueError(f"routed experts: activation={activation!r}")
        self.activation, self.has_correction = activation, bool(correction)
        self.groups, self.keep, self.route_scale, self.identity = int(groups), int(keep), float(route_scale), int(identity)
        if group_mark not in ("max", "top2_sum"):
            raise ValueError(f"routed experts: group_mark={group_mark!r}")
        self.group_top = 2 if group_mark == "top2_sum" else 1
        self.routes = self.E + self.identity                       # the router's outputs
        if self.identity < 0 or self.top > self.routes:
            raise ValueError(f"routed experts: top_k={self.top} of {self.routes} router outputs, {self.identity} of them identities")
        if not (1 <= self.keep <= self.groups and self.routes % self.groups == 0
                and self.keep * (self.routes // self.groups) >= self.top):
            raise ValueError(f"routed experts: {self.groups} groups over {self.routes} router outputs, {self.keep} kept, "
                             f"cannot give {self.top} choices")

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {"router": ParamSpec((self.routes, self.hidden))}
        if self.has_correction:
            s["correction"] = ParamSpec((self.routes,), kind="vector", init="normal")
        for e in range(self.E):
            if self.activation == "swiglu":
                s[f"e{e}.gate"] = ParamSpec((self.F, self.hidden))
            s[f"e{e}.up"] = ParamSpec((self.F, self.hidden))
            s[f"e{e}.down"] = ParamSpec((self.hidden, self.F))
        if self.SF:
            s["shared.up"] = ParamSpec((self.SF, self.hidden))
            s["shared.down"] = ParamSpec((self.hidden, self.SF))
            if self.shared_gate:
                s["shared.sg"] = ParamSpec((1, self.hidden))
        return s

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        self.w_router = params.pop("router")
        self.up_layout = self.activation
        if self.activation == "swiglu":
            gates, ups = [params.pop(f"e{e}.gate") for e in range(self.E)], [params.pop(f"e{e}.up") for e in range(self.E)]
            if gates[0].dtype == torch.bfloat16 and self.F % 8 == 0 and self.hidden % 8 == 0 and hasattr(self.rt.k, "moe_grouped"):
                # an expert's first matrix in sixteens of 8 gate rows and the 8 matching up rows: the layout whose
                # product writes silu(gate) * up from its epilogue
                from ..kernels import interleave_gate_up
                self.w_up = torch.stack([interleave_gate_up(g, u) for g, u in zip(gates, ups)]).contiguous()
                self.up_layout = "swiglu_interleaved"
            else:
                # its gate rows, then its up rows
                self.w_up = torch.stack([torch.cat([g, u]) for g, u in zip(gates, ups)]).contiguous()
        else:
            self.w_up = torch.stack([params.pop(f"e{e}.up") for e in range(self.E)]).contiguous()
        # (the choice adds it to fp32 scores: widened once, exactly)
        self.correction = params.pop("correction").float().contiguous() if self.has_correction else None
        self.w_down = torch.stack([params.pop(f"e{e}.down") for e in range(self.E)]).contiguous()
        self.w_sup = self.w_sdown = self.w_sg = None
        if self.SF:
            self.w_sup, self.w_sdown = params.pop("shared.up"), params.pop("shared.down")
            self.w_sg = params.pop("shared.sg") if self.shared_gate else None
            self.check_products(shared_up=self.w_sup, shared_down=self.w_sdown)
        # bfloat16: the router's logits (and the shared gate's) as one product of the library with fp32 sums and fp32
        # output (bf16 operands multiply exactly in fp32); the 32-bit path keeps the FFMA router kernel
        self.w_route = None
        if self.w_router.dtype == torch.bfloat16 and self.hidden % 8 == 0 and hasattr(self.rt.k, "moe_choose"):
            rows = [self.w_router] + ([self.w_sg.reshape(1, self.hidden)] if self.w_sg is not None else [])
            self.w_route = torch.cat(rows).contiguous()

    def tensors(self) -> Dict[str, torch.Tensor]:
        out = {"router": self.w_router}
        if self.has_correction:
            out["correction"] = self.correction
        for e in range(self.E):
            if self.up_layout == "swiglu_interleaved":
                gu = self.w_up[e].view(self.F // 8, 2, 8, self.hidden)
                out[f"e{e}.gate"], out[f"e{e}.up"] = gu[:, 0].reshape(self.F, self.hidden), gu[:, 1].reshape(self.F, self.hidden)
            elif self.activation == "swiglu":
                out[f"e{e}.gate"], out[f"e{e}.up"] = self.w_up[e, :self.F], self.w_up[e, self.F:]
            else:
                out[f"e{e}.up"] = self.w_up[e]
            out[f"e{e}.down"] = self.w_down[e]
        if self.SF:
            out["shared.up"], out["shared.down"] = self.w_sup, self.w_sdown
            if self.shared_gate:
                out["shared.sg"] = self.w_sg
        return out

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        rt, k = self.rt, self.rt.k
        T = x.shape[0]
        idx = rt.ws.get("moe.idx", (T, self.top), torch.int32)
        wgt = rt.ws.get("moe.wgt", (T, self.top), torch.float32)
        gate = rt.ws.get("moe.gate", (T,), torch.float32) if self.shared_gate else None
        if self.w_route is not None:
            logits = rt.ws.get("moe.logits", (T, self.w_route.shape[0]), torch.float32)
            k.linear(logits, x, self.w_route)
            k.moe_choose(idx, wgt, logits, self.routes, self.top, gate, self.score, self.renormalize, self.correction,
                         self.groups, self.keep, self.route_scale, self.group_top)
        else:
            k.moe_route(idx, wgt, x, self.w_router, self.top, gate, self.w_sg, self.score, self.renormalize,
                        self.correction, self.groups, self.keep, self.route_scale, self.group_top)
        grouped = self.up_layout == "swiglu_interleaved" or (self.activation == "relu2" and not self.identity)
        if (grouped and T > 16 and rt.dtype == torch.bfloat16 and self.F % 8 == 0 and self.hidden % 8 == 0
                and x.stride(0) % 8 == 0 and hasattr(k, "moe_grouped")):
            # many tokens: pairs sorted by expert, each expert's rows as tiles of one grouped product
            k.moe_grouped(residual, x, self.w_up, self.w_down, idx, wgt, self.scale_input,
                          activation=self.up_layout, identity=bool(self.identity))
        else:
            # few tokens (and the 32-bit path): every (token, choice) streams its expert's matrices
            act = rt.ws.get("moe.act", (T, self.top, self.F), rt.dtype)
            k.moe_up(act, x, self.w_up, idx, wgt, self.scale_input, self.up_layout)
            k.moe_down(residual, act, self.w_down, idx, x if self.identity else None, wgt)
        if self.SF:
            u = rt.ws.get("moe.shared_u", (T, self.SF), rt.dtype)
            k.linear(u, x, self.w_sup)
            a = rt.ws.get("moe.shared_a", (T, self.SF), rt.dtype)
            k.relu2_scale(a, u, gate)
            k.linear(residual, a, self.w_sdown, accumulate=True, defer=True)     # a norm reads the stream next
