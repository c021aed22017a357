"""Token embedding and the output head.

hidden = E[token, :], no scale (src/architectures/impl/qwen3/block.zig:16-18);
logits = W_out y in fp32, where W_out is the embedding table when the model is
tied (src/architectures/impl/qwen3/block.zig:43-46, src/tuner/compile.zig:170-174).
"""
from __future__ import annotations

from typing import Any, Dict, Mapping, Optional

import torch

from ..registry import NORMS, lookup, register_embedding, register_head
from .base import ParamSpec, Part


@register_embedding("token_embedding")
class TokenEmbedding(Part):
    """``norm``: a registered norm ({"kind": ..., its parameters}) that the looked-up rows pass
    through before they become the stream; its tensors are ``norm.<local name>``."""

    def __init__(self, vocab_size: int, hidden_size: int, norm: Optional[Mapping[str, Any]] = None):
        self.vocab, self.hidden = int(vocab_size), int(hidden_size)
        self.weight: Optional[torch.Tensor] = None
        self.norm = None
        if norm is not None:
            norm = dict(norm)
            self.norm = lookup(NORMS, "norm", norm.pop("kind"))(size=self.hidden, **norm)

    def param_specs(self) -> Dict[str, ParamSpec]:
        s = {"weight": ParamSpec((self.vocab, self.hidden))}
        if self.norm is not None:
            s.update({"norm." + n: p for n, p in self.norm.param_specs().items()})
        return s

    def attach(self, rt) -> None:
        super().attach(rt)
        if self.norm is not None:
            self.norm.attach(rt)

    def bind(self, params: Dict[str, torch.Tensor]) -> None:
        self.weight = params["weight"]
        if self.norm is not None:
            self.norm.bind({n[5:]: t for n, t in params.items() if n.startswith("norm.")})

    def tensors(self) -> Dict[str, torch.Tensor]:
        out = {"weight": self.weight}
        if self.norm is not None:
            out.update({"norm." + n: t for n, t in self.norm.tensors().items()})
        return out

    def forward(self, out: torch.Tensor, ids: torch.Tensor) -> None:
        if self.norm is None:
            self.rt.k.embed(out, self.weight, ids)
            return
        raw = self.rt.ws.get("embed.raw", out.shape, torch.float32)
        self.rt.k.embed(raw, self.weight, ids)
        self.norm.forward(out, raw)


@register_head("lm_head")
class LMHead(Part):
    def __init__(self, vocab_size: int, hidden_size: int, tied: bool):
        self.vocab, self.hidden, self.tied = int(vocab_size), int(hidden_size), bool(tied)
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
