"""What a model is made of: specifications (data), part interfaces and the registries of part kinds.

A model is a `ModelSpec`: an embedding, a list of `LayerSpec`s (each names the kind and the
parameters of its block arrangement, mixer, feed-forward and norms), an `order` in which layers
run (a layer may be named twice; a call may read the cache that an earlier call owns), a final
norm and an output head.  Nothing in a part knows which model it is in: sizes and constants
arrive as constructor parameters, tensor names arrive through `PartSpec.weights`.

The reference hard-wires this structure in one file per model
(core/src/model_executor/models/llama/llama.rs:276-536); its `trait Model`
(core/src/model_executor/models/model.rs:44-52) is the only shared interface.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Optional, Tuple, Union

import torch

# ----------------------------------------------------------------------------- specifications


@dataclass
class PartSpec:
    """kind: a name in the registry of its family; params: constructor keywords;
    weights: logical weight name -> checkpoint tensor name, or a list of names whose tensors
    are concatenated along dimension 0 (q, k, v into one matrix; gate, up into one)."""
    kind: str
    params: Dict[str, Any] = field(default_factory=dict)
    weights: Dict[str, Union[str, List[str]]] = field(default_factory=dict)


@dataclass
class LayerSpec:
    """block: kind of arrangement; parts: role in that arrangement -> PartSpec."""
    block: str
    parts: Dict[str, PartSpec]
    block_params: Dict[str, Any] = field(default_factory=dict)


@dataclass
class LayerCall:
    """One entry of the run order.  `layer` indexes ModelSpec.layers.  `cache_of`: index of an
    EARLIER entry of the order whose cache this call reads instead of owning one."""
    layer: int
    cache_of: Optional[int] = None


@dataclass
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_model_len: int
    embedding: PartSpec
    layers: List[LayerSpec]
    order: List[LayerCall]
    final_norm: PartSpec
    lm_head: PartSpec
    eos_token_ids: List[int] = field(default_factory=list)
    ignored_weights: List[str] = field(default_factory=list)     # regular expressions of tensors to skip


@dataclass
class WeightSpec:
    """Shapes of the source tensors (concatenated along dim 0, in order).  `keep_fp32`: a source
    stored in 32-bit stays float32 even when the run dtype is bfloat16 (norm weights, biases)."""
    shapes: List[Tuple[int, ...]]
    keep_fp32: bool = False


@dataclass(frozen=True)
class KVCacheSpec:
    """What a mixer needs of the paged cache: per token and layer 2 * num_kv_heads * head_dim
    values; window None keeps all keys, window w keeps the last w."""
    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None


@dataclass(frozen=True)
class StateSpec:
    """Per-request state of fixed size that a mixer keeps across steps (float32 unless told)."""
    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


# ----------------------------------------------------------------------------- what a step hands to the parts


@dataclass
class CacheGroupView:
    """Block tables of the live requests for one group of layers."""
    block_table: torch.Tensor      # int32 [n_seqs, max_blocks] on the device, -1 where no page
    block_size: int


@dataclass
class LayerCache:
    """The cache of one call of the order, as its mixer sees it."""
    kv: Optional[torch.Tensor] = None          # [pages, 2, kv_heads, block_size, head_dim]
    group: Optional[int] = None                # index into StepContext.groups
    state: Optional[torch.Tensor] = None       # [slots, *StateSpec.shape]
    owner: bool = True                         # False: read another call's cache, write nothing


@dataclass
class StepContext:
    """One batch: `n_tokens` tokens of `n_seqs` requests, each request's tokens consecutive."""
    n_tokens: int
    n_seqs: int
    dtype: torch.dtype
    device: torch.device
    token_ids: torch.Tensor        # int32 [n_tokens]
    positions: torch.Tensor        # int32 [n_tokens] absolute position of each token
    token_seq: torch.Tensor        # int32 [n_tokens] index of the token's request in this batch
    cu_q: torch.Tensor             # int32 [n_seqs + 1] token offsets of the requests
    ctx_len: torch.Tensor          # int32 [n_seqs] tokens in the cache after this step
    state_slot: torch.Tensor       # int32 [n_seqs]
    groups: List[CacheGroupView]
    # host copies for launch geometry and for parts written on the host side
    q_lens: List[int] = field(default_factory=list)
    ctx_lens: List[int] = field(default_factory=list)
    state_slots: List[int] = field(default_factory=list)
    error_flag: Optional[torch.Tensor] = None
    # geometry of the batch for kernels that treat single tokens and portions apart
    decode_seq_ids: Optional[torch.Tensor] = None      # int32: requests that bring one token
    n_decode_seqs: int = 0
    q_tile_seq: Optional[torch.Tensor] = None          # int32: request of each 64-token tile of a longer portion
    q_tile_q0: Optional[torch.Tensor] = None           # int32: first token of the tile inside its portion
    n_q_tiles: int = 0
    q_tile128_seq: Optional[torch.Tensor] = None       # the same in tiles of 128 tokens
    q_tile128_q0: Optional[torch.Tensor] = None
    n_q_tiles128: int = 0
    extras: Dict[str, Any] = field(default_factory=dict)   # per-step scratch that kernels share across layers

    @property
    def max_q_len(self) -> int:
        return max(self.q_lens) if self.q_lens else 0

    @property
    def max_ctx_len(self) -> int:
        return max(self.ctx_lens) if self.ctx_lens else 0

    @property
    def decode_only(self) -> bool:
        return self.max_q_len <= 1


Q_TILE = 64      # query tokens per tile in StepContext.q_tile_*

# ----------------------------------------------------------------------------- interfaces


class Part:
    """Base of every part.  A part declares its weights, receives them, and computes."""

    # True when the part's work in a step of single tokens depends on the batch's size only (no value read back
    # to the host, no launch whose shape depends on the data): only then may such a step be captured as a CUDA
    # graph and replayed.  A part that does not say so keeps its model on eager steps.
    graph_safe = False

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {}

    def set_weights(self, tensors: Dict[str, torch.Tensor]) -> None:
        for k, v in tensors.items():
            setattr(self, k, v)

    def prepare(self, dtype: torch.dtype, device: torch.device) -> None:
        """Builds device constants (tables) once the run dtype and device are known."""

    def activation_width(self) -> int:
        """How many values per token the part keeps alive at its widest (its intermediate tensors); the engine
        sizes the memory it leaves free for a step's activations from the widest part."""
        return 0


class Norm(Part):
    # True when the norm is a factor per row times a weight per column, so that the products around it can share its
    # work (`NormAfter`, `Prenormed`); such a norm has `weight`, `eps`, `hidden_size` and `finish`.
    splittable = False

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def forward_residual(self, x: torch.Tensor, res: Optional[torch.Tensor]) -> Tuple[torch.Tensor, torch.Tensor]:
        """res' = res + x in float32 (res None: res' = x); returns (norm(res'), res').  A splittable norm is also
        handed its own `Prenormed` (the add is done): it returns it as it is."""
        raise NotImplementedError


@dataclass
class NormAfter:
    """What a block hands to a mixer or feed-forward that says `fuses_norm`: the norm that follows the part and the
    residual stream.  If the part's last product can, it adds its result to `res` itself, does the first half of the
    norm and returns a `Prenormed` instead of a tensor (`linear.matmul_tn_residual`).  A step of a few tokens saves a
    kernel and a round trip through memory between two products that way."""
    norm: Norm
    res: torch.Tensor


@dataclass
class Prenormed:
    """A norm's output before the division: `x` = residual x norm weight (bfloat16), `sumsq` [rows, parts] float32
    partial sums of the squares of the residual's rows.  The factor 1 / sqrt(sum / width + eps) is common to a row, so
    a product that takes a Prenormed (a part that says `takes_prenormed`; `linear.matmul_tn`) applies it to its
    sums.  `norm.finish(p)` gives the ordinary normed tensor."""
    x: torch.Tensor
    sumsq: torch.Tensor
    eps: float
    width: int
    norm: Norm
    res: torch.Tensor


class PositionEncoding(Part):
    def apply(self, ctx: StepContext, q: torch.Tensor, k: Optional[torch.Tensor], n_q_heads: int, n_kv_heads: int,
              head_dim: int) -> None:
        """Encodes positions into q and k in place ([n, heads * head_dim] views)."""
        raise NotImplementedError

    def fused_rotary(self) -> Optional[Tuple[torch.Tensor, int, bool]]:
        """(inv_freq float32 [rot_dim / 2], rot_dim, is_neox) when the encoding is a rotation that the
        cache-write kernel can apply itself; None otherwise."""
        return None

    def score_slopes(self) -> Optional[torch.Tensor]:
        """float32 [query heads] when the encoding is a bias on the attention scores that grows with distance,
        slope * (key position - query position); None otherwise."""
        return None


class Mixer(Part):
    # takes_prenormed: `forward` accepts a `Prenormed` as h.  fuses_norm: `forward` accepts `then=NormAfter(...)` and
    # may return a `Prenormed`.  A part that says neither is always given and asked for plain tensors.
    takes_prenormed = False
    fuses_norm = False

    def cache_spec(self) -> Optional[KVCacheSpec]:
        return None

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def forward(self, ctx: StepContext, h: torch.Tensor, cache: LayerCache) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    takes_prenormed = False     # as for a mixer
    fuses_norm = False

    def forward(self, ctx: StepContext, h: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of parts.  `parts` maps role names to built parts; the block says which
    roles it needs in `ROLES` (role -> family)."""
    ROLES: Dict[str, str] = {}

    def __init__(self, parts: Dict[str, Part], **params):
        self.parts = parts

    @property
    def mixer(self) -> Optional[Mixer]:
        return self.parts.get("mixer")  # type: ignore[return-value]

    def forward(self, ctx: StepContext, x: torch.Tensor, res: Optional[torch.Tensor], cache: LayerCache
                ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
        """(x, res) -> (x, res): x is the branch output not yet added, res the float32 residual sum."""
        raise NotImplementedError

    def entry(self) -> Optional[Tuple[Norm, Part]]:
        """(the norm that the block's input meets first, the part that reads that norm's output), for the block that
        runs before this one and says `fuses_next_norm`: its `forward` is then called with `next_entry=` this pair
        and may return a `Prenormed` for that norm as x.  None (the default): the block wants a plain tensor."""
        return None

    fuses_next_norm = False


# ----------------------------------------------------------------------------- registries

FAMILIES = ("mixer", "feed_forward", "norm", "position_encoding", "block", "embedding", "linear")
_REGISTRY: Dict[str, Dict[str, Callable[..., Any]]] = {f: {} for f in FAMILIES}


def register_part(family: str, kind: str):
    """Class decorator: `@register_part("mixer", "paged_attention")`."""
    if family not in _REGISTRY:
        raise KeyError(f"unknown part family {family!r} (families: {', '.join(FAMILIES)})")

    def deco(cls):
        _REGISTRY[family][kind] = cls
        return cls
    return deco


def part_class(family: str, kind: str):
    try:
        return _REGISTRY[family][kind]
    except KeyError:
        known = ", ".join(sorted(_REGISTRY.get(family, {})))
        raise KeyError(f"no {family} of kind {kind!r} is registered (known: {known})") from None


def build_part(family: str, spec: PartSpec) -> Part:
    params = dict(spec.params)
    # a nested PartSpec is built first; its key names its family
    # (e.g. params["position_encoding"] of an attention mixer)
    nested = []
    for k, v in list(params.items()):
        if isinstance(v, PartSpec):
            params[k] = build_part(k, v)
            nested.append((params[k], v))
    part = part_class(family, spec.kind)(**params)
    part.nested_parts = nested        # parts with weights of their own are loaded like any other
    return part


def with_nested(part: Part, spec: PartSpec):
    """(part, spec) and, after it, every part nested inside it with its own spec."""
    yield part, spec
    for child, child_spec in getattr(part, "nested_parts", ()):
        yield from with_nested(child, child_spec)
