"""What a part of a model is: the interfaces, the registries, and what a step hands to a part.

A model is put together from parts that know nothing of the model they are in:

- a *norm* turns the float32 residual stream into activations of the compute type;
- a *mixer* lets rows of one sequence see earlier rows (attention here), through memory
  the cache gives it: token-indexed pages, or per-sequence state of fixed size;
- a *feed-forward* maps rows to rows;
- a *position encoding* is a parameter of a mixer (rotary tables) or acts on embeddings;
- a *block* arranges norms, a mixer and a feed-forward around the residual stream.

Each kind has a registry from a name to a class.  A model's specification
(:class:`ModelSpec`) names a kind and its parameters for every layer separately, plus the
order in which layers run, so two layers of one model may differ in every part.

Mixers and feed-forwards *add* their result into the residual stream they are given:
that lets their last product fuse the addition.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, List, Mapping, Optional, Tuple

import torch


# ------------------------------------------------------------------------------- registries

class Registry:
    """Name -> class of one kind of part."""

    def __init__(self, what: str):
        self.what = what
        self._items: Dict[str, Callable] = {}

    def register(self, name: str, item: Optional[Callable] = None):
        def put(obj):
            if name in self._items and self._items[name] is not obj:
                raise ValueError(f"{self.what} '{name}' is already registered")
            self._items[name] = obj
            return obj

        return put if item is None else put(item)

    def unregister(self, name: str) -> None:
        self._items.pop(name, None)

    def get(self, name: str) -> Callable:
        if name not in self._items:
            raise KeyError(f"no {self.what} named '{name}' (known: {sorted(self._items)})")
        return self._items[name]

    def names(self) -> List[str]:
        return sorted(self._items)


NORMS = Registry("norm")
MIXERS = Registry("mixer")
FEED_FORWARDS = Registry("feed-forward")
POSITION_ENCODINGS = Registry("position encoding")
BLOCKS = Registry("block")
EMBEDDINGS = Registry("embedding")
HEADS = Registry("head")


# --------------------------------------------------------------------------- specifications

@dataclass(frozen=True)
class PartSpec:
    """One part of one layer: which kind, with which sizes and constants, and the prefix
    its tensors carry in the model folder."""

    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)
    prefix: str = ""


class LayerSpec:
    """One layer: the block that arranges it and the block's parts by the role each plays
    in it.  Which roles a block has (and which registry builds each) is the block's own
    business (``Block.ROLES``): ``LayerSpec("prenorm", norm1=..., mixer=..., norm2=...,
    feed_forward=...)`` for the built-in block, other names for another."""

    def __init__(self, block: str, parts: Optional[Mapping[str, PartSpec]] = None, **named: PartSpec):
        self.block = block
        self.parts: Dict[str, PartSpec] = dict(parts or {})
        self.parts.update(named)
        for role, spec in self.parts.items():
            if not isinstance(spec, PartSpec):
                raise TypeError(f"layer part '{role}' must be a PartSpec, got {type(spec).__name__}")

    def __repr__(self) -> str:
        return f"LayerSpec({self.block!r}, {self.parts!r})"


@dataclass(frozen=True)
class RunSpec:
    """One entry of the order in which layers run.  ``layer`` indexes ModelSpec.layers and
    may occur in several entries (shared weights).  ``memory_of`` names an earlier entry
    whose cache and state this run reads instead of keeping its own."""

    layer: int
    memory_of: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    schedule: Tuple[RunSpec, ...]
    final_norm: PartSpec
    head: PartSpec
    stop_ids: Tuple[int, ...] = ()
    # A position encoding that acts on the stream right after the embedding (its
    # ``on_embeddings``), with tensors of its own if it wants any; None for models whose
    # positions live inside their mixers (rotary tables).
    position: Optional[PartSpec] = None


# -------------------------------------------------------------------------- declared tensors

@dataclass(frozen=True)
class TensorSpec:
    """A tensor a part wants from the model folder.

    ``role`` decides its type on the device: "matrix" operands take the compute type
    (bfloat16 when serving, float32 on the 32-bit path); "vector" (norm weights and the
    like) is float32 on both paths, which is exact for what a folder stores in bfloat16 and
    keeps what it stores in 32-bit as it is; "index" tables are int32.
    ``init`` tells the random-weights mode how to fill it.
    """

    shape: Tuple[int, ...]
    role: str = "matrix"
    init: str = "normal"
    optional: bool = False


# ------------------------------------------------------------------------------ the runtime

@dataclass
class Runtime:
    """Where and in which precision a model runs."""

    device: torch.device
    dtype: torch.dtype  # compute type: torch.bfloat16 or torch.float32
    max_positions: int = 0  # most positions any sequence can reach (0: the model's own limit)

    @property
    def is_f32(self) -> bool:
        return self.dtype == torch.float32


@dataclass
class CacheNeed:
    """Token-indexed memory a mixer wants for each cached position, as planes: plane i
    keeps ``planes[i] = (heads, width)`` values of the compute type a position, stored a
    page of 64 positions at a time as [pages, heads, 64, width].  Attention asks for two
    equal planes (keys, values); a mixer that caches one latent vector a token asks for
    one plane (1, width); planes may differ in shape.  ``window`` > 0 if only that many
    latest positions are ever read.  Runs with equal needs share one storage group."""

    planes: Tuple[Tuple[int, int], ...]
    window: int = 0

    def __post_init__(self):
        self.planes = tuple((int(h), int(w)) for h, w in self.planes)
        if not self.planes or any(h <= 0 or w <= 0 for h, w in self.planes):
            raise ValueError(f"a cache need wants at least one plane of positive sizes, got {self.planes}")

    @staticmethod
    def keys_values(kv_heads: int, head_dim: int, window: int = 0) -> "CacheNeed":
        """Keys and values of ``kv_heads`` heads of ``head_dim`` a position."""
        return CacheNeed(((kv_heads, head_dim), (kv_heads, head_dim)), window)

    def key(self) -> Tuple:
        return (self.planes, self.window)

    def values_per_token(self) -> int:
        return sum(h * w for h, w in self.planes)


@dataclass
class StateNeed:
    """Per-sequence memory of fixed size a mixer wants: one tensor of ``shape`` and
    ``dtype`` per slot, zeroed when the slot is handed out."""

    shape: Tuple[int, ...]
    dtype: torch.dtype = torch.float32


@dataclass
class RunMemory:
    """What one run of a layer may read and write in the cache this step."""

    planes: Tuple[torch.Tensor, ...] = ()       # one [pages, heads, PAGE, width] tensor per plane of the mixer's CacheNeed
    page_table: Optional[torch.Tensor] = None   # [slots, max_pages] int32
    state: Optional[torch.Tensor] = None        # [slots, *StateNeed.shape]
    writes: bool = True                         # False when reading another run's memory

    @property
    def k_pages(self) -> Optional[torch.Tensor]:
        """The first plane: keys, for a mixer that asked for keys and values."""
        return self.planes[0] if self.planes else None

    @property
    def v_pages(self) -> Optional[torch.Tensor]:
        return self.planes[1] if len(self.planes) > 1 else None


@dataclass
class StepContext:
    """One step's batch, flattened to rows.  Row r is the token at position row_pos[r] of
    the sequence in slot row_slot[r]; a negative slot marks a padding row, which must
    change nothing that lives past the step.  Sequence s owns rows
    seq_rows[s] .. seq_rows[s + 1]; before this step its slot held seq_start[s] tokens.
    The device tensors may be longer than ``rows`` / ``seqs`` says (they are reused)."""

    rows: int
    seqs: int
    tokens: torch.Tensor        # [rows] int32
    row_pos: torch.Tensor       # [rows] int32
    row_slot: torch.Tensor      # [rows] int32
    seq_rows: torch.Tensor      # [seqs + 1] int32
    seq_slot: torch.Tensor      # [seqs] int32
    seq_start: torch.Tensor     # [seqs] int32
    max_new: int                # most rows any one sequence brings
    max_total: int              # most positions any one sequence reaches after this step
    decode: bool                # every sequence brings exactly one row
    # Host copies, for parts that plan on the host.
    host_seq_rows: Tuple[int, ...] = ()
    host_seq_slot: Tuple[int, ...] = ()
    host_seq_start: Tuple[int, ...] = ()
    extras: Dict[str, Any] = field(default_factory=dict)


# ------------------------------------------------------------------------------- interfaces

class Part:
    """Base of every part.  A part is built from its PartSpec's params on the host, says
    which tensors it wants, and receives them (already on the device, already in the type
    their role asks for) in :meth:`load`."""

    # False for a part whose forward plans on the host from this step's lengths (ctx.host_*):
    # the engine then runs every step eagerly instead of replaying a captured graph.
    graph_safe = True

    def __init__(self, **params: Any):
        self.params = params

    def tensors(self) -> Dict[str, TensorSpec]:
        """Names (relative to the part's prefix) and shapes of the tensors it wants."""
        return {}

    def load(self, tensors: Dict[str, torch.Tensor], rt: Runtime) -> None:
        self.rt = rt


class Norm(Part):
    def forward(self, residual: torch.Tensor, out: torch.Tensor, gather: Optional[torch.Tensor] = None) -> None:
        """out = norm(residual rows) in the compute type; ``gather`` picks rows."""
        raise NotImplementedError


class PositionEncoding(Part):
    """Either hook may do nothing.  ``rotary`` gives a mixer what it needs to rotate
    queries and keys; ``on_embeddings`` may add to the stream right after the embedding."""

    def rotary(self) -> Optional["RotaryTable"]:
        return None

    def on_embeddings(self, residual: torch.Tensor, ctx: StepContext) -> None:
        return None


@dataclass
class RotaryTable:
    cos_sin: torch.Tensor   # [positions, head_dim // 2, 2] float32: (cos, sin) of position * inv_freq
    pairing: int            # 0: (i, i + d/2); 1: (2i, 2i + 1)


class Mixer(Part):
    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def rollback_state(self, state: torch.Tensor, slot: int, length: int) -> bool:
        """A sequence is cut back to ``length`` positions.  Token-indexed memory goes back
        by its length alone, but per-sequence state has already absorbed the positions that
        are dropped.  A mixer that can put ``state[slot]`` back to what it was after
        ``length`` positions (from snapshots of its own, or because the state can be
        rebuilt) does so and returns True.  The default, False, makes the engine refuse the
        cut with a CacheError, so that state from the future is never left in place."""
        return False

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext, mem: RunMemory) -> None:
        """residual[:rows] += mix(x); x is [rows, hidden] in the compute type.

        A mixer with ``graph_safe = True`` is replayed from a captured graph on decode
        steps.  The engine warms the step up and captures it with every row marked as
        padding (slot -1), so a forward must leave memory and state untouched for such rows;
        real rows then run exactly once a step."""
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        """residual[:rows] += f(x)."""
        raise NotImplementedError


class Embedding(Part):
    def forward(self, ctx: StepContext, residual: torch.Tensor) -> None:
        """residual[r] = embedding of ctx.tokens[r], as float32."""
        raise NotImplementedError

    def table(self) -> Optional[torch.Tensor]:
        """The [vocab, hidden] table, for a head tied to it."""
        return None


class Head(Part):
    def forward(self, x: torch.Tensor, out: torch.Tensor, tied: Optional[torch.Tensor]) -> None:
        """out [rows, vocab] float32 = scores of normalised rows x."""
        raise NotImplementedError


class Block(Part):
    """Arranges parts around the residual stream.  ``ROLES`` names the parts a block is
    made of and the registry that builds each; a LayerSpec must give exactly these.  The
    built parts are attributes of the block under their role names."""

    ROLES: Dict[str, Registry] = {}

    def __init__(self, parts: Mapping[str, Part], hidden_size: int):
        super().__init__()
        self.parts: Dict[str, Part] = dict(parts)
        self.hidden_size = hidden_size
        for role, part in self.parts.items():
            setattr(self, role, part)

    @classmethod
    def build(cls, spec: LayerSpec, hidden_size: int) -> "Block":
        missing = [r for r in cls.ROLES if r not in spec.parts]
        unexpected = [r for r in spec.parts if r not in cls.ROLES]
        if missing or unexpected:
            raise ValueError(f"block '{spec.block}' is made of {sorted(cls.ROLES)}; missing {sorted(missing)}, unexpected {sorted(unexpected)}")
        return cls({role: cls.ROLES[role].get(spec.parts[role].kind)(**dict(spec.parts[role].params)) for role in cls.ROLES}, hidden_size)

    def named_parts(self, spec: LayerSpec):
        """(tensor-name prefix, part) of every part of this block, in the order of ROLES."""
        for role in self.ROLES:
            yield spec.parts[role].prefix, self.parts[role]

    def memory_part(self) -> Optional[Mixer]:
        """The part whose cache_need() / state_need() the cache serves for a run of this
        block, and that receives the run's RunMemory: its mixer, if it has one."""
        part = self.parts.get("mixer")
        return part if isinstance(part, Mixer) else None

    def forward(self, residual: torch.Tensor, ctx: StepContext, mem: RunMemory, rt: Runtime) -> None:
        raise NotImplementedError
