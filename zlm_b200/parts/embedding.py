"""Token embedding and the output head.

hidden = E[token, :], no scale (src/architectures/impl/qwen3/block.zig:16-18);
logits = W_out y in fp32, where W_out is the embedding table when the model is
tied (src/architectures/impl/qwen3/block.zig:43-46, src/tuner/compile.zig:170-174).
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from ..registry import NORMS, lookup, register_embedding, register_head
from .base import LayerIO, ParamSpec, Part, StateRequest, StepContext


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    """``norm``: a registered norm ({"kind": ..., its parameters}) that the looked-up rows pass
    through before they become the stream; its tensors are ``norm.<local name>``.

    ``scale``: the looked-up row is multiplied by it.  ``pair`` ({"buckets", "mul_prev", "mul_cur"}): a second table
    ``pair`` of buckets + 1 rows is added, looked up by the token and the token before it, row
    (prev * mul_prev + cur * mul_cur) mod buckets, and its last row for a sequence's first token.  The token before a
    step's first one is state of the sequence (one int32 per slot, ``state_request``)."""

    def __init__(self, vocab_size: int, hidden_size: int, norm: Optional[Mapping[str, Any]] = None, scale: float = 1.0,
                 pair: Optional[Mapping[str, int]] = None):
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.weight: Optional[torch.Tensor] = None
        self.scale = float(scale)
        self.pair = None
        self.pair_table: Optional[torch.Tensor] = None
        if pair is not None:
            self.pair = (int(pair["buckets"]), int(pair["mul_prev"]), int(pair["mul_cur"]))
            if self.pair[0] <= 0 or min(self.pair[1:]) < 0:
                raise ValueError(f"embedding: pair table with buckets={self.pair[0]}, multipliers {self.pair[1:]}")
        # whether ``forward`` wants the step's context and the part's state beside the token ids
        self.uses_step = self.pair is not None
        self.norm = None
        if norm is not None:
            norm = dict(norm)
            self.norm = lookup(NORMS, "norm", norm.pop("kind"))(size=self.hidden, **norm)

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {"weight": ParamSpec((self.vocab, self.hidden))}
        if self.pair is not None:
            s["pair"] = ParamSpec((self.pair[0] + 1, self.hidden))
        if self.norm is not None:
            s.update({"norm." + n: p for n, p in self.norm.param_specs().items()})
        return s

    def attach(self, rt) -> None:
        super().attach(rt)
        if self.norm is not None:
            self.norm.attach(rt)

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((), torch.int32) if self.pair is not None else None

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        self.weight = params["weight"]
        self.pair_table = params.get("pair")
        if self.norm is not None:
            self.norm.bind({n[5:]: t for n, t in params.items() if n.startswith("norm.")})

    def tensors(self) -> Dict[str, torch.Tensor]:
        out = {"weight": self.weight}
        if self.pair is not None:
            out["pair"] = self.pair_table
        if self.norm is not None:
            out.update({"norm." + n: t for n, t in self.norm.tensors().items()})
        return out

    def _lookup(self, out: torch.Tensor, ids: torch.Tensor, ctx: Optional[StepContext], io: Optional[LayerIO]) -> None:
        k = self.rt.k
        if self.pair is None and self.scale == 1.0:
            k.embed(out, self.weight, ids)
        elif self.pair is None:
            k.embed_scaled(out, self.weight, ids, self.scale)
        else:
            if ctx is None or io is None or io.state is None:
                raise ValueError("embedding: the pair table needs the step's context and the sequences' state")
            k.embed_scaled(out, self.weight, ids, self.scale, self.pair_table, *self.pair, plan=ctx, prev_state=io.state)

    def forward(self, out: torch.Tensor, ids: torch.Tensor, ctx: Optional[StepContext] = None,
                io: Optional[LayerIO] = None) -> None:
        if self.norm is None:
            self._lookup(out, ids, ctx, io)
            return
        raw = self.rt.ws.get("embed.raw", out.shape, torch.float32)
        self._lookup(raw, ids, ctx, io)
        self.norm.forward(out, raw)


@register_head("lm_head")
class LMHead(Part):
    def __init__(self, vocab_size: int, hidden_size: int, tied: bool, logit_scale: float = 1.0, softcap: float = 0.0):
        """``logit_scale``: the logits are multiplied by it (in fp32, after the product).  ``softcap``: the logits
        become softcap * tanh(logits / softcap) (0: no cap)."""
        self.vocab, self.hidden, self.tied = int(vocab_size), int(hidden_size), bool(tied)
        self.logit_scale, self.softcap = float(logit_scale), float(softcap)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        # a tied checkpoint may still carry a copy of the table under the head's name
        return {"weight": ParamSpec((self.vocab, self.hidden), ignorable=self.tied)}

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = params["weight"]
            self.check_products(weight=self.weight)

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table
        self.check_products(weight=self.weight)

    def forward(self, logits: torch.Tensor, x: torch.Tensor) -> None:
        """logits [R, vocab] fp32 = x [R, hidden] . W^T"""
        self.rt.k.linear(logits, x, self.weight)
        if self.logit_scale != 1.0:
            self.rt.k.scale_(logits, self.logit_scale)
        if self.softcap > 0.0:
            self.rt.k.softcap_(logits, self.softcap)
