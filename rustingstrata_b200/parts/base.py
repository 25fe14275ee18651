"""Interfaces that every part implements, and the objects parts are handed.

The reference passes raw device addresses through a ~70-method backend trait
(src/backend.rs:98-443) and hard-codes the layer loop per architecture
(src/gpu_model.rs:3072-3423).  Here a part is a small object with three duties:

* say which checkpoint tensors it wants (:meth:`Part.tensor_needs`) and take them
  (:meth:`Part.load`);
* say what it keeps between steps (:meth:`Mixer.cache_need`, :meth:`Mixer.state_need`);
* run on the tokens of one step (:meth:`forward`), reading the step's metadata from a
  :class:`StepContext`.

A part never looks at the model it is in.  Sizes and constants come from
``PartSpec.params``; buffers come from the :class:`Runtime`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Mapping, Optional, Sequence, Tuple

import numpy as np
import torch

from .spec import CacheNeed, PartSpec, StateNeed, TensorNeed


class Runtime:
    """What a part may use at build time: element type, device, limits, shared scratch buffers."""

    def __init__(self, dtype: torch.dtype, device: torch.device, max_batch_tokens: int, max_seqs: int,
                 max_logit_rows: int, page_size: int, max_positions: int, pool_tokens: int):
        self.dtype = dtype
        self.device = device
        self.max_batch_tokens = max_batch_tokens
        self.max_seqs = max_seqs
        self.max_logit_rows = max_logit_rows
        self.page_size = page_size
        self.max_positions = max_positions
        self.pool_tokens = pool_tokens          # tokens one cache group's page pool holds
        self._buffers: Dict[str, torch.Tensor] = {}
        self._wanted: Dict[str, tuple] = {}
        self._shared: Dict[Any, Any] = {}

    @property
    def precise(self) -> bool:
        return self.dtype == torch.float32

    def scratch(self, name: str, rows: int, width: int, dtype: Optional[torch.dtype] = None) -> None:
        """Declares a [rows, width] buffer shared by every part that asks for the same name and element
        type (sized for the largest request).  It is allocated at its first use; contents do not survive
        from one part call to the next."""
        dtype = dtype or self.dtype
        key = f"{name}:{dtype}"
        r, w = self._wanted.get(key, (0, 0, None))[:2]
        self._wanted[key] = (max(r, rows), max(w, width), dtype)
        cur = self._buffers.get(key)
        if cur is not None and (cur.shape[0] < rows or cur.shape[1] < width):
            del self._buffers[key]

    def get_scratch(self, name: str, dtype: Optional[torch.dtype] = None) -> torch.Tensor:
        key = f"{name}:{dtype or self.dtype}"
        cur = self._buffers.get(key)
        if cur is None:
            rows, width, dt = self._wanted[key]
            cur = torch.empty((rows, width), dtype=dt, device=self.device)
            self._buffers[key] = cur
        return cur

    def shared(self, key, make):
        """One object per key for the whole model (e.g. a rotation table shared by all layers)."""
        if key not in self._shared:
            self._shared[key] = make()
        return self._shared[key]


@dataclass
class HostBatch:
    """The step's batch as the host knows it (numpy int32 arrays of length n_seqs unless noted)."""
    n_tokens: int
    n_seqs: int
    q_lens: np.ndarray            # tokens of each sequence in this step
    kv_lens: np.ndarray           # keys of each sequence after this step
    q_start: np.ndarray           # [n_seqs + 1] first token row of each sequence
    state_slots: np.ndarray       # state slot of each sequence
    first_step: np.ndarray        # 1 where the sequence has no earlier tokens
    page_size: int
    max_blocks: List[int]         # per cache group: width of the block tables of this step
    bucketed: bool = False        # the step may be captured in a CUDA graph: host scalars that become launch
                                  # shapes must be rounded up to buckets so that later steps can replay it


@dataclass
class CallInfo:
    """Where one mixer of one entry of the run order keeps its things (what ``Mixer.forward`` is handed)."""
    index: int                            # position in the run order
    layer: int
    role: str = "mixer"                   # the mixer's role in its layer
    cache_group: Optional[int] = None     # page pool ("cache group") of the cache this call uses
    cache: Optional[torch.Tensor] = None  # [pages, 2, n_kv, page_size, head_dim] view of that cache
    writes_cache: bool = True             # False when the call reads another call's cache
    state: Optional[torch.Tensor] = None  # [max_seqs, numel] per-request state of this call, in the type it asked for


@dataclass
class LayerCallInfo:
    """One entry of the run order: the layer it runs and the storage of each of the layer's mixers, by role."""
    index: int
    layer: int
    mixers: Dict[str, CallInfo] = field(default_factory=dict)


@dataclass
class StepContext:
    """Device-side metadata of one step; all index tensors are int32."""
    n_tokens: int
    n_seqs: int
    n_logit_rows: int
    token_ids: torch.Tensor        # [T]
    positions: torch.Tensor        # [T, n_streams]: column 0 is the token's place in its sequence (and in the cache);
                                   # further columns are position streams that the request supplied, for position
                                   # encodings that follow something other than the token count (equal to column
                                   # 0 where none were given).  One column for every model whose parts ask for one.
    seq_of_token: torch.Tensor     # [T] index of the token's sequence within this step
    q_start: torch.Tensor          # [S + 1]
    kv_len: torch.Tensor           # [S]
    state_slots: torch.Tensor      # [S]
    logit_rows: torch.Tensor       # [R] token rows whose logits are wanted
    block_tables: List[torch.Tensor]   # per cache group [S, max_blocks]
    status: torch.Tensor           # [1] error bits set by kernels
    host: HostBatch
    plans: Dict[Any, Dict[str, Any]] = field(default_factory=dict)   # per plan key: device arrays + host scalars
    # A product into the residual stream may leave its last step (adding up partial sums) to the next reader of the
    # stream.  ``may_owe``: set by the block around a mixer's or feed-forward's call when that reader can take it;
    # ``owed``: what the mixer or feed-forward left (an object with finish()), taken by the block for the next norm;
    # ``next_block_takes_owed``: set by the model before each block, for the block's last product.
    may_owe: bool = False
    owed: Any = None
    next_block_takes_owed: bool = False


class Part:
    """Base of all parts."""
    category = ""
    kind = ""
    # Whether forward() only enqueues work whose shape and addresses depend on the step's layout alone (no read of
    # device results on the host, no host loop over the batch's contents).  A step is captured into a CUDA graph
    # only if every part of the model says so; a part that needs the host says False and its model runs eagerly.
    capturable = True
    # Whether the part touches the step's tensors through the kernel launchers of ``kernels.ops`` only (no torch
    # arithmetic on them).  Only then may the engine let those launchers hold back the products of a small decode step and
    # send them off as one chained kernel: work done behind the launchers' back would not see what they still hold.
    chain_safe = False

    def __init__(self, spec: PartSpec, runtime: Runtime):
        self.spec = spec
        self.runtime = runtime

    # -- weights
    def tensor_needs(self) -> Dict[str, TensorNeed]:
        """Checkpoint tensor name → shape and role, for every tensor this part reads."""
        return {}

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        """Takes its tensors (already on the device, in the element types the loader kept)."""

    # -- per-step planning (host side, before any kernel of the step)
    def plan_key(self):
        """A hashable key if the part needs per-step index arrays; parts with equal keys share one plan."""
        return None

    def build_plan(self, batch: HostBatch) -> Dict[str, Any]:
        """int32 numpy arrays (uploaded with the step's metadata) and host scalars for this step."""
        return {}


class Mixer(Part):
    """Token mixer: reads the normed activations ``h`` [T, hidden] of the step and adds its output
    into the float32 residual stream ``residual`` [T, hidden] in place."""

    def cache_need(self) -> Optional[CacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, call: CallInfo) -> None:
        raise NotImplementedError


class FeedForward(Part):
    """Per-token feed-forward: reads ``h`` [T, hidden], adds its output into ``residual`` in place."""

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> None:
        raise NotImplementedError


class Norm(Part):
    """Normalisation of the float32 residual stream into the activation type.

    A norm whose ``takes_owed`` is true has a keyword ``owed`` in ``forward``: a sum still owed to ``x`` (see
    StepContext), which it adds while it reads the rows."""
    takes_owed = False

    def forward(self, x: torch.Tensor, out: torch.Tensor, n_rows: int, rows: Optional[torch.Tensor] = None) -> None:
        raise NotImplementedError


class PositionEncoding(Part):
    """What a mixer needs to encode positions; the mixer's kernels consume it.

    ``cos_sin`` / ``n_rot``: a rotation table [positions, cos(n_rot/2) | sin(n_rot/2)] (None / 0: no rotation);
    ``n_streams``: how many position values per token the step must carry for this part (1: the token's place in its
    sequence is all it needs); ``stream``: which of them its table is indexed by; ``score_slopes``: None, or float32
    [heads] on the device: slope of head h times (key position - query position) is added to every scaled score."""
    n_streams = 1
    stream = 0
    cos_sin = None
    n_rot = 0
    score_slopes = None


class Block(Part):
    """Arrangement of a layer's parts around the residual stream.

    ``roles`` (class attribute) names what the arrangement is made of: role → part category.  The model builds the
    parts a layer's description lists, checks them against ``roles`` (every role listed must be known; every role
    not in ``optional`` must be there) and hands them over as a mapping; the block is free in what it does with
    them in ``forward``.  Roles of category "mixer" are the ones that can own a cache or state: the model asks each
    for its needs, and ``forward`` finds each one's storage in ``call.mixers[role]``."""
    roles: Mapping[str, str] = {}
    optional: Tuple[str, ...] = ()

    def __init__(self, spec, runtime, parts: Mapping[str, Part]):
        super().__init__(spec, runtime)
        self.parts: Dict[str, Part] = dict(parts)

    @classmethod
    def check_roles(cls, given) -> None:
        known = dict(cls.roles)
        extra = [r for r in given if r not in known and not cls._is_position_role(r)]
        lacking = [r for r in known if r not in given and r not in cls.optional]
        if extra or lacking:
            raise ValueError(f"block '{cls.kind}' is made of {sorted(known)}"
                             + (f"; unknown roles: {sorted(extra)}" if extra else "")
                             + (f"; missing roles: {sorted(lacking)}" if lacking else ""))

    @classmethod
    def _is_position_role(cls, role: str) -> bool:
        return role == "position" or (role.endswith("_position") and cls.roles.get(role[: -len("_position")]) == "mixer")

    @classmethod
    def category_of(cls, role: str) -> str:
        return "position" if cls._is_position_role(role) else cls.roles[role]

    def mixers(self) -> Dict[str, Mixer]:
        return {r: p for r, p in self.parts.items() if self.roles.get(r) == "mixer"}

    @property
    def first_reader_takes_owed(self) -> bool:
        """Whether the first thing this block does with the residual stream is a norm that takes an owed sum; only
        then may the block before it leave one."""
        return False

    def forward(self, residual: torch.Tensor, ctx: StepContext, call: "LayerCallInfo") -> None:
        raise NotImplementedError

    @staticmethod
    def norm_of_stream(norm: Norm, residual: torch.Tensor, out: torch.Tensor, ctx: StepContext) -> None:
        """norm(residual) → out for the step's tokens, settling what is owed to the stream on the way."""
        owed, ctx.owed = ctx.owed, None
        if owed is not None and getattr(norm, "takes_owed", False):
            norm.forward(residual, out, ctx.n_tokens, owed=owed)
            return
        if owed is not None:
            owed.finish()
        norm.forward(residual, out, ctx.n_tokens)
