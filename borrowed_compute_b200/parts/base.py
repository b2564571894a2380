"""What a part of a model is: the interfaces, the registries, and what a step hands to a part.

A model is put together from parts that know nothing of the model they are in:

- a *norm* turns the float32 residual stream into activations of the compute type;
- a *mixer* lets rows of one sequence see earlier rows (attention here), through memory
  the cache gives it: token-indexed pages, or per-sequence state of fixed size;
- a *feed-forward* maps rows to rows;
- a *position encoding* is a parameter of a mixer (rotary tables) or acts on embeddings;
- a *short convolution* mixes a few neighbouring rows of one sequence on every channel and
  keeps the last of them as per-sequence state;
- a *block* arranges norms, a mixer and a feed-forward around the residual stream;
- a *junction* acts on the residual stream between two layers (where a stretch of layers is
  entered again, say) and may read the embedding's output.

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
CONVOLUTIONS = Registry("short convolution")
BLOCKS = Registry("block")
JUNCTIONS = Registry("junction")
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
    whose cache and state this run reads instead of keeping its own.  ``enter`` = (junction,
    pass) runs ModelSpec.junctions[junction] on the stream right before this run, telling it
    the number of the pass that starts here (a stretch of layers that runs several times)."""

    layer: int
    memory_of: Optional[int] = None
    enter: Optional[Tuple[int, int]] = None


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
    # (name, shape) of tensors a folder may hold although no part reads them (the norm of a
    # branch that a layer leaves out, say): tolerated when present, never asked for.
    tolerated: Tuple[Tuple[str, Tuple[int, ...]], ...] = ()
    # Parts that act on the stream between layers; a RunSpec's ``enter`` names one.
    junctions: Tuple[PartSpec, ...] = ()


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
    latest positions are ever read; ``chunk`` > 0 if a position only ever reads those of its
    own chunk of that many positions (counted from position 0), so that whole chunks behind
    the newest one can be let go.  ``keep_first`` > 0 if the first that many positions of a sequence stay readable
    whatever the window (they are never let go).  Runs with equal needs share one storage group."""

    planes: Tuple[Tuple[int, int], ...]
    window: int = 0
    chunk: int = 0
    keep_first: int = 0

    def __post_init__(self):
        self.planes = tuple((int(h), int(w)) for h, w in self.planes)
        if not self.planes or any(h <= 0 or w <= 0 for h, w in self.planes):
            raise ValueError(f"a cache need wants at least one plane of positive sizes, got {self.planes}")

    @staticmethod
    def keys_values(kv_heads: int, head_dim: int, window: int = 0, value_dim: Optional[int] = None, chunk: int = 0,
                    keep_first: int = 0) -> "CacheNeed":
        """Keys of ``kv_heads`` heads of ``head_dim`` a position, and values of ``value_dim``
        (default: the same width)."""
        return CacheNeed(((kv_heads, head_dim), (kv_heads, head_dim if value_dim is None else value_dim)), window, chunk, keep_first)

    def key(self) -> Tuple:
        return (self.planes, self.window, self.chunk, self.keep_first)

    def values_per_token(self) -> int:
        return sum(h * w for h, w in self.planes)


@dataclass
class StateNeed:
    """Per-sequence memory of fixed size a mixer wants: one tensor of ``shape`` and
    ``dtype`` per slot, zeroed when the slot is handed out.  ``dtype`` None asks for the
    compute type of the runtime (bfloat16 when serving, float32 on the 32-bit path)."""

    shape: Tuple[int, ...]
    dtype: Optional[torch.dtype] = torch.float32


@dataclass
class RunMemory:
    """What one run of a layer may read and write in the cache this step."""

    planes: Tuple[torch.Tensor, ...] = ()       # one [pages, heads, PAGE, width] tensor per plane of the mixer's CacheNeed
    page_table: Optional[torch.Tensor] = None   # [slots, max_pages] int32
    state: Optional[torch.Tensor] = None        # [slots, *StateNeed.shape]: the mixer's own
    writes: bool = True                         # False when reading another run's memory
    # State of the block's other parts, by the role each plays in the block ("conv": ...).
    states: Dict[str, torch.Tensor] = field(default_factory=dict)

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

    def more_state_needs(self) -> Dict[str, StateNeed]:
        """Further per-sequence state by a name of the mixer's choosing (the last inputs of a
        convolution inside it, say); a run finds each in ``RunMemory.states["mixer." + name]``.
        Like the block's other state it cannot be put back after a cut, save the cut to 0."""
        return {}

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


class ShortConvolution(Part):
    """A causal convolution over a few rows of each sequence, channel by channel.  Its
    state (the last inputs of every sequence) lives in the cache like a mixer's."""

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, h: torch.Tensor, out: torch.Tensor, ctx: StepContext, state: Optional[torch.Tensor], writes: bool = True) -> None:
        """out = conv(h) for the rows of the step, each sequence continuing from ``state``;
        rows of padding sequences (slot -1) change nothing that outlives the step."""
        raise NotImplementedError


class Junction(Part):
    """Acts on the residual stream between two layers."""

    needs_embedding = False     # whether forward wants the embedding's output of the step's rows

    def forward(self, residual: torch.Tensor, embedded: Optional[torch.Tensor], ctx: StepContext, number: int) -> None:
        """Changes residual[:rows] in place; ``number`` counts the passes that have entered here."""
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
    made of and the registry that builds each; a LayerSpec must give exactly these, save
    those of ``OPTIONAL``, which a layer may leave out (the attribute is then None).  The
    built parts are attributes of the block under their role names."""

    ROLES: Dict[str, Registry] = {}
    OPTIONAL: Tuple[str, ...] = ()

    def __init__(self, parts: Mapping[str, Part], hidden_size: int):
        super().__init__()
        self.parts: Dict[str, Part] = dict(parts)
        self.hidden_size = hidden_size
        for role in self.OPTIONAL:
            setattr(self, role, None)
        for role, part in self.parts.items():
            setattr(self, role, part)

    @classmethod
    def build(cls, spec: LayerSpec, hidden_size: int) -> "Block":
        missing = [r for r in cls.ROLES if r not in spec.parts and r not in cls.OPTIONAL]
        unexpected = [r for r in spec.parts if r not in cls.ROLES]
        if missing or unexpected:
            raise ValueError(f"block '{spec.block}' is made of {sorted(cls.ROLES)}; missing {sorted(missing)}, unexpected {sorted(unexpected)}")
        return cls({role: cls.ROLES[role].get(spec.parts[role].kind)(**dict(spec.parts[role].params))
                    for role in cls.ROLES if role in spec.parts}, hidden_size)

    def named_parts(self, spec: LayerSpec):
        """(tensor-name prefix, part) of every part of this block, in the order of ROLES."""
        for role in self.ROLES:
            if role in self.parts:
                yield spec.parts[role].prefix, self.parts[role]

    def state_needs(self) -> Dict[str, StateNeed]:
        """Per-sequence state that parts of this block other than its mixer want, by role,
        and what the mixer wants beside its own state ("mixer." + the mixer's name for it);
        a run of the block finds each in ``RunMemory.states``."""
        mixer = self.memory_part()
        return {} if mixer is None else {"mixer." + name: need for name, need in mixer.more_state_needs().items()}

    def rollback_states(self, states: Mapping[str, torch.Tensor], slot: int, length: int) -> bool:
        """Like ``Mixer.rollback_state`` for the state of ``state_needs``: True if every one
        was put back to what it was after ``length`` positions.  A block without such state
        has nothing to put back."""
        return not states

    def memory_part(self) -> Optional[Mixer]:
        """The part whose cache_need() / state_need() the cache serves for a run of this
        block, and that receives the run's RunMemory: its mixer, if it has one."""
        part = self.parts.get("mixer")
        return part if isinstance(part, Mixer) else None

    def forward(self, residual: torch.Tensor, ctx: StepContext, mem: RunMemory, rt: Runtime) -> None:
        raise NotImplementedError
