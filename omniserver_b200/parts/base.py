"""Interfaces of the parts a decoder is put together from.

A model is a list of layers; a layer is a block that arranges a mixer
(attention here), a feed-forward and norms; mixers may use a position
encoding.  Every part takes its sizes and constants as constructor
parameters and names its checkpoint tensors itself; none knows which model it
is in.  Parts are looked up by name in the registries below, so a new kind of
part is one class and one ``register_*`` call and needs no change to the
framework's files.

The reference has the same roles as fixed classes (RMSNorm, Attention, MLP,
DecoderLayer in omniserve/model/qwen2_llm.py:39-157); here they are chosen by
the configuration layer by layer.
"""

from __future__ import annotations

import abc
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------- parameters
@dataclass(frozen=True)
class ParamSpec:
    """One tensor a part owns, and where it comes from in a checkpoint.

    ``sources`` are checkpoint names relative to the part's prefix; several
    sources are concatenated along dim 0 in that order (the reference fuses
    q/k/v and gate/up this way, omniserve/model/qwen2_llm.py:207-216).
    ``kind``: "float" tensors take the engine's dtype unless the file stores
    them in 32-bit; "int" tensors become int32.
    ``init``: what the random-weights mode draws: "normal", "ones" (norm
    weights: ones plus optional noise) or "zeros".
    """

    attr: str
    sources: Tuple[str, ...]
    shapes: Tuple[Tuple[int, ...], ...]
    kind: str = "float"
    init: str = "normal"

    @property
    def shape(self) -> Tuple[int, ...]:
        first = self.shapes[0]
        return (sum(s[0] for s in self.shapes),) + tuple(first[1:])


# --------------------------------------------------------------------------- cache needs
@dataclass(frozen=True)
class KVCacheNeed:
    """Paged keys and values: ``window`` None keeps all keys, else the last ``window``."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size (a row of ``shape`` per request slot).

    ``shared`` state is one field for the whole model under ``name`` (all
    parts asking for it get the same tensor); otherwise every layer entry
    gets a field of its own.
    """

    name: str
    shape: Tuple[int, ...]
    dtype: torch.dtype
    shared: bool = False


@dataclass
class CacheBinding:
    """What the cache manager hands a mixer for one entry of the layer schedule.

    ``k_cache``/``v_cache``: this entry's pages ``[num_pages, kv_heads, page_size, head_dim]``.
    ``group``: index of the page group (block tables and slot maps are per group).
    ``writes``: False when the entry reads another entry's cache and must not write.
    ``state``: name -> tensor ``[num_slots, *shape]`` of per-request state.
    """

    group: Optional[int] = None
    k_cache: Optional[torch.Tensor] = None
    v_cache: Optional[torch.Tensor] = None
    writes: bool = True
    state: Dict[str, torch.Tensor] = field(default_factory=dict)


# --------------------------------------------------------------------------- part base classes
class Part(abc.ABC):
    """A piece of a layer with tensors of its own."""

    #: checkpoint prefix relative to the model's prefix, e.g. "layers.3.self_attn."
    prefix: str = ""

    def param_specs(self) -> List[ParamSpec]:
        return []

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        """Receive the loaded tensors, keyed by ParamSpec.attr."""
        for k, v in tensors.items():
            setattr(self, k, v)


class Norm(Part):
    @abc.abstractmethod
    def forward_add(self, x: torch.Tensor, residual: Optional[torch.Tensor], out_dtype: torch.dtype
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
        """residual <- residual + x (or x when None), in 32-bit; returns (norm(residual), residual)."""

    @abc.abstractmethod
    def forward_add_rows(self, x: torch.Tensor, residual: torch.Tensor, rows: torch.Tensor,
                         out_dtype: torch.dtype) -> torch.Tensor:
        """norm(residual[rows] + x[rows]) for the given rows only; nothing is written back."""

    def fused_linear(self, x: torch.Tensor, residual: Optional[torch.Tensor], linear: Any, out_dtype: torch.dtype
                     ) -> Optional[Tuple[torch.Tensor, torch.Tensor]]:
        """(linear(norm(residual + x)), new residual) in one kernel where this norm has one for these
        operands (a decode step's few rows), else None: the caller then runs ``forward_add`` and the
        projection. ``linear`` has ``weight`` [N, K] and ``bias`` (or None)."""
        return None

    def rms_operands(self) -> Optional[Tuple[torch.Tensor, float]]:
        """(weight, eps) if this norm is y = r / sqrt(mean(r^2) + eps) * weight with r = residual + x and
        nothing else, for a part whose kernel computes that norm itself; None for any other norm."""
        return None


@dataclass
class RotaryOperands:
    """What a rotary encoding hands a mixer for one step: cos and sin ``[T, rot_dim / 2]`` in fp32 for the
    step's tokens. Element d < rot_dim / 2 of a head is rotated together with element d + rot_dim / 2;
    elements from ``rot_dim`` on are left alone."""

    cos: torch.Tensor
    sin: torch.Tensor
    rot_dim: int


class PositionEncoding(Part):
    """Turns positions into what a mixer applies to its queries and keys.

    The engine knows nothing of an encoding's positions: it carries ``position_columns`` rows of integers
    per token where a request gives them, writes the state rows ``request_state`` returns into the
    request's slot, and asks ``positions_for`` which columns to send with a span of tokens.
    """

    #: rows of integers per token that a request may give with its prompt (0: the encoding takes none)
    position_columns: int = 0

    def state_needs(self) -> List[StateNeed]:
        return []

    def request_state(self, given: Optional[Any], num_prompt_tokens: int) -> Dict[str, Sequence[Any]]:
        """When a request takes (or, after preemption, takes again) its state slot: the values of this
        encoding's state fields for it, by field name. ``given``: the positions that came with the
        prompt, ``[position_columns, num_prompt_tokens]``, or None. Fields not named start at zero."""
        return {}

    def positions_for(self, given: Optional[Any], num_prompt_tokens: int, start: int, stop: int) -> Optional[Any]:
        """The columns ``[position_columns, stop - start]`` to send with tokens [start, stop) of a request
        (its prompt followed by what it generated), or None where the encoding finds the positions
        itself from its state. The default sends what was given and can say nothing past the prompt."""
        if given is None or start >= num_prompt_tokens:
            return None
        if stop > num_prompt_tokens:
            raise ValueError("this position encoding cannot continue given positions past the prompt")
        return given[:, start:stop]

    @abc.abstractmethod
    def prepare(self, ctx: "Any", state: Dict[str, torch.Tensor]) -> Any:
        """Once per step: per-token tables shared by every layer that uses this encoding."""

    def rotary(self, tables: Any) -> Optional[RotaryOperands]:
        """The step's tables as a rotation of element pairs (d, d + rot_dim / 2), which the attention
        kernels can apply themselves while they write the cache; None for any other encoding."""
        return None

    def apply(self, ctx: "Any", tables: Any, qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int
              ) -> None:
        """For an encoding that is no such rotation: changes the queries and keys in ``qkv``
        ``[T, (num_heads + 2 num_kv_heads) * head_dim]`` in place. The default leaves them alone."""

    def finish_step(self, ctx: "Any", state: Dict[str, torch.Tensor]) -> None:
        """Once per step after all layers ran (advance cursors and the like)."""


class Mixer(Part):
    """Mixes information across the tokens of a request (attention, or anything with state)."""

    def cache_needs(self) -> List[object]:
        return []

    @abc.abstractmethod
    def forward(self, ctx: "Any", x: torch.Tensor, binding: CacheBinding) -> torch.Tensor:
        """x [T, hidden] -> [T, hidden]; reads and writes its cache through ``binding``."""

    def forward_prenorm(self, ctx: "Any", x: torch.Tensor, residual: Optional[torch.Tensor], norm: Norm,
                        binding: CacheBinding) -> Tuple[torch.Tensor, torch.Tensor]:
        """forward(norm(residual + x)) and the new residual stream. A mixer whose first projection can
        take the norm into its kernel (``norm.fused_linear``) overrides this; the default runs both."""
        h, residual = norm.forward_add(x, residual, ctx.act_dtype)
        return self.forward(ctx, h, binding), residual


class FeedForward(Part):
    @abc.abstractmethod
    def forward(self, ctx: "Any", x: torch.Tensor) -> torch.Tensor:
        """x [T, hidden] -> [T, hidden], token by token."""

    def forward_prenorm(self, ctx: "Any", x: torch.Tensor, residual: Optional[torch.Tensor], norm: Norm
                        ) -> Tuple[torch.Tensor, torch.Tensor]:
        """forward(norm(residual + x)) and the new residual stream (see ``Mixer.forward_prenorm``)."""
        h, residual = norm.forward_add(x, residual, ctx.act_dtype)
        return self.forward(ctx, h), residual


class Block(abc.ABC):
    """The arrangement of norms, mixer and feed-forward in one layer."""

    mixer: Mixer

    @abc.abstractmethod
    def parts(self) -> List[Part]:
        ...

    @abc.abstractmethod
    def forward(self, ctx: "Any", x: torch.Tensor, residual: Optional[torch.Tensor],
                binding: CacheBinding) -> Tuple[torch.Tensor, torch.Tensor]:
        """One layer on the step's tokens; returns (branch output, residual stream)."""


# --------------------------------------------------------------------------- registries
@dataclass(frozen=True)
class PartSpec:
    """A part chosen by name with its constructor parameters."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)

    def __hash__(self) -> int:  # params may hold lists
        return hash((self.kind, repr(sorted(self.params.items()))))


class Registry:
    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Callable[..., Any]] = {}

    def register(self, name: str, factory: Callable[..., Any]) -> None:
        self._items[name] = factory

    def build(self, spec: PartSpec, **extra: Any) -> Any:
        if spec.kind not in self._items:
            raise KeyError(f"unknown {self.what} {spec.kind!r}; known: {sorted(self._items)}")
        return self._items[spec.kind](**spec.params, **extra)

    def names(self) -> List[str]:
        return sorted(self._items)

    def __contains__(self, name: str) -> bool:
        return name in self._items


NORMS = Registry("norm")
POSITIONS = Registry("position encoding")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
BLOCKS = Registry("block")


def register_norm(name: str, factory: Callable[..., Norm]) -> None:
    NORMS.register(name, factory)


def register_position_encoding(name: str, factory: Callable[..., PositionEncoding]) -> None:
    POSITIONS.register(name, factory)


def register_mixer(name: str, factory: Callable[..., Mixer]) -> None:
    MIXERS.register(name, factory)


def register_feed_forward(name: str, factory: Callable[..., FeedForward]) -> None:
    FEED_FORWARDS.register(name, factory)


def register_block(name: str, factory: Callable[..., Block]) -> None:
    BLOCKS.register(name, factory)
