"""``MultiHeadAttention`` with the reference's constructor options and call
signatures (packages/runntime/src/core/nn/layers.ts:886-956): a thin module
that holds the optional per-head sink logits and forwards to sdpa/sdpaPacked.
It takes already-projected q/k/v and applies no score scale."""
from __future__ import annotations

from typing import Optional

from .ops import sdpa, sdpaPacked
from .value import Value, ValueMeta


class Parameter:
    """A named weight slot; ``value`` is set when weights are loaded."""

    def __init__(self, shape: ValueMeta, value: Optional[Value] = None, pinned: bool = False):
        self.shape, self._value, self.pinned = shape, value, pinned

    @property
    def value(self) -> Value:
        if self._value is None:
            raise RuntimeError("Parameter.value: not loaded")
        return self._value

    def set(self, value: Value) -> None:
        if value.shape.elems != self.shape.elems or value.shape.dtype != self.shape.dtype:
            raise ValueError(
                f"Parameter.set: expected {self.shape.elems} {self.shape.dtype} elems, got "
                f"{value.shape.elems} {value.shape.dtype}")
        self._value = value


class MultiHeadAttention:
    """opts: {qHeads, kvHeads, headDim, windowLeft, windowRight, sinks?}."""

    def __init__(self, opts: dict):
        self.opts = dict(opts)
        # pinned: attention sinks are f32 in every kernel variant
        self.sinks: Optional[Parameter] = (
            Parameter(ValueMeta(opts["qHeads"], "f32", (opts["qHeads"],)), None, True)
            if opts.get("sinks") else None)

    def parameters(self):
        return {"sinks": self.sinks} if self.sinks is not None else {}

    def _opts(self, call: Optional[dict]) -> dict:
        call = call or {}
        o = self.opts
        return {
            "qHeads": o["qHeads"], "kvHeads": o["kvHeads"], "headDim": o["headDim"],
            "windowLeft": o["windowLeft"], "windowRight": o["windowRight"],
            "qPosOffset": call.get("qPosOffset"),
            "sinks": self.sinks.value if self.sinks is not None else None,
            "segments": call.get("segments"), "maxSegment": call.get("maxSegment"),
        }

    def forward(self, q: Value, k: Value, v: Value, call: Optional[dict] = None) -> Value:
        return sdpa(q, k, v, self._opts(call))

    def forwardPacked(self, qkv: Value, call: Optional[dict] = None) -> Value:
        """Self-attention over one fused qkv tensor read in place; same result
        as forward(q, k, v) on the sliced blocks."""
        return sdpaPacked(qkv, self._opts(call))

    __call__ = forward
