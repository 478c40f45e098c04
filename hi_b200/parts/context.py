"""What the step function hands to the parts: the batch of one step, and a mixer's cache."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

import torch


@dataclass
class StepContext:
    """One step: N new tokens of S requests, flat. All tensors live on the device.

    Request ``s`` contributes ``n_new[s]`` consecutive tokens at positions
    ``start_pos[s] ..``; rows ``cu_seqlens[s] .. cu_seqlens[s+1]`` of every [N, ...] tensor
    are its tokens. ``slots[s]`` is the request's fixed-size state slot.
    """

    n_tokens: int
    n_seqs: int
    tokens: torch.Tensor          # int32 [N]
    positions: torch.Tensor       # int32 [N]  absolute position of each token
    seq_of_token: torch.Tensor    # int32 [N]  row of the block tables / index into slots
    cu_seqlens: torch.Tensor      # int32 [S+1]
    slots: torch.Tensor           # int32 [S]
    start_pos: List[int]          # host copies
    n_new: List[int]
    slot_ids: List[int]
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)   # group -> int32 [S, width]
    page_size: int = 0
    max_context: int = 0          # longest start_pos + n_new in the step
    tap: Optional[Callable[[str, torch.Tensor], None]] = None   # debug: parts report named tensors
    # debug: choices a part is told to take instead of its own, by the name it reports them under
    # (the router's expert ids, int32 [N, k] in the step's flat token order)
    forced: Optional[Dict[str, torch.Tensor]] = None
    # mixed steps only: flat rows of the requests that bring ONE token (int64 [D]) and the longest
    # context among them; None when the step is all portions or all single tokens
    decode_rows: Optional[torch.Tensor] = None
    decode_max_context: int = 0
    # what parts of one forward pass hand to later parts of the same pass (emptied at its start):
    # an arrangement that needs the results of earlier layers keeps them here
    scratch: Dict[str, object] = field(default_factory=dict)

    @property
    def max_new(self) -> int:
        return max(self.n_new) if self.n_new else 0


@dataclass
class CacheView:
    """The cache slot of one schedule entry, as its mixer sees it."""

    group: Optional[int] = None                  # page group (None: no paged cache)
    k_pages: Optional[torch.Tensor] = None       # [pages, kv_heads, page_size, head_dim]
    v_pages: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None         # [max_slots, *state_shape]
    writes: bool = True                          # False: read another entry's cache, do not append
    slot: Optional[int] = None                   # the cache slot's number (a key for per-pass scratch)
    block_state: Optional[torch.Tensor] = None   # [max_slots, n] float32: fixed-size state of the block arrangement


@dataclass
class Pending:
    """A sub-layer's output that has not yet been added to the residual stream: a dense part
    (engine dtype or float32, [N, H]) and/or the routed experts' rows (float32 [N*k, H] in
    expert-sorted order, with the slot of every (token, rank) entry). The next norm adds all of
    it in one pass."""

    dense: Optional[torch.Tensor] = None
    dense2: Optional[torch.Tensor] = None            # a second dense part (two sub-layers side by side)
    routed: Optional[torch.Tensor] = None
    slot_of_entry: Optional[torch.Tensor] = None
    top_k: int = 0
    entry_weights: Optional[torch.Tensor] = None     # float32 [N*k]: factors of the routed rows in the sum

    def materialize(self, n_tokens: int) -> torch.Tensor:
        """The sum as one float32 tensor, for a consumer that is not a norm."""
        from ..kernels import ops

        if self.dense2 is not None:
            total = torch.zeros((n_tokens, self.dense.shape[1]), dtype=torch.float32, device=self.dense.device)
            ops.stream_add(total, self.dense, self.dense2)
            if self.routed is None:
                return total
            return ops.moe_combine(self.routed, self.slot_of_entry, total, n_tokens, self.top_k, self.entry_weights)
        if self.routed is None:
            return self.dense
        return ops.moe_combine(self.routed, self.slot_of_entry, self.dense, n_tokens, self.top_k, self.entry_weights)


@dataclass
class GatedPending:
    """What a block with gated, side-by-side sub-layers leaves for the next norm: the sub-layers'
    results with what their gates' sigmoids take (``terms``: (delta, gate | None), [N, W] each), and,
    where the model hands on a weighted average of all layer results so far, the history of those
    results (float32 [entries, N, W], ``filled`` of them written) with this layer's weights
    (float32 [filled + 1]). The norm that takes it adds the gated terms into the stream, stores the sum
    as the next entry, averages, and normalises, in one kernel."""

    terms: list
    history: Optional[torch.Tensor] = None
    filled: int = 0
    mix: Optional[torch.Tensor] = None


@dataclass
class HyperPending:
    """What a block with a residual stream of several copies leaves for the next norm: a sub-layer's result
    (``delta``: a tensor or a :class:`Pending`) and the coefficients it enters the copies with,
    x_t <- sum_s mix[s, t] x_s + mult * out_coef[t] * delta. The stream handed on beside it is the tensor of the
    copies, float32 [N, S, W]; the norm that takes it updates them and reads its own input off them in one kernel."""

    delta: object
    mix: torch.Tensor            # float32 [S, S], indexed [from, to]
    out_coef: torch.Tensor       # float32 [S]
    mult: float = 1.0
