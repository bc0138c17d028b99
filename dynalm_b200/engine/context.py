"""The per-step metadata every part sees, and the view of the cache a mixer is handed."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class CacheView:
    """One run-order entry's share of the cache for the current step.

    kind "pages": `arrays` are [pages, page_size, *entry_shape] tensors (keys and values for
    attention) and `block_table` is int32 [request slots, max_blocks]: page of position p of the request in
    slot s = block_table[s, p // page_size] (-1 where a windowed group has given the page back, and where the
    request has no page yet). The table lives on the device; a step sends only what changed.
    kind "state": `arrays[0]` is [slots, *state_shape]; the step's request r owns row
    `ctx.state_slots[r]`.
    """

    kind: str
    arrays: List[torch.Tensor]
    page_size: int = 0
    block_table: Optional[torch.Tensor] = None


@dataclass
class StepContext:
    """One step: a batch of (request, its next tokens), flattened.

    Row i of the step is token `token_ids[i]` at position `positions[i]` of the step's request
    `row_request[i]`, whose slot (the row of the block tables and of state arrays that it owns for as long as it
    lives) is `row_slot[i]`; request r's rows are q_start[r] .. q_start[r+1]-1, consecutive positions from
    pos_start[r]; after the step it holds kv_len[r] = pos_start[r] + rows tokens. All tensors are
    int32 on the device; the `h_` lists are the same values on the host for parts that plan launches.
    """

    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    row_request: torch.Tensor
    row_slot: torch.Tensor
    q_start: torch.Tensor
    pos_start: torch.Tensor
    kv_len: torch.Tensor
    state_slots: torch.Tensor
    logit_rows: torch.Tensor
    num_logit_rows: int
    h_q_len: List[int] = field(default_factory=list)
    h_pos_start: List[int] = field(default_factory=list)
    h_state_slots: List[int] = field(default_factory=list)
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)   # cache group -> [request slots, max_blocks]
    decode_only: bool = False        # every request brings exactly one token
    max_q_len: int = 0
    max_kv_len: int = 0
    # per-step scratch that parts share. A part's step plan (see StepShape in engine/step.py) is found under its name
    # as (the plan's integers on the device, what its `fill` returned); parts may add entries of their own.
    extras: Dict[str, object] = field(default_factory=dict)
