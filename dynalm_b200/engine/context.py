"""The per-step metadata every part sees, and the view of the cache a mixer is handed."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch


@dataclass
class CacheView:
    """One run-order entry's share of the cache for the current step.

    kind "pages": `arrays` are [pages, page_size, *entry_shape] tensors (keys and values for
    attention) and `block_table` is int32 [requests, max_blocks]: page of position p of the step's
    request r = block_table[r, p // page_size] (-1 where a windowed group has given the page back).
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
    `row_request[i]`; request r's rows are q_start[r] .. q_start[r+1]-1, consecutive positions from
    pos_start[r]; after the step it holds kv_len[r] = pos_start[r] + rows tokens. All tensors are
    int32 on the device; the `h_` lists are the same values on the host for parts that plan launches.
    """

    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor
    positions: torch.Tensor
    row_request: torch.Tensor
    q_start: torch.Tensor
    pos_start: torch.Tensor
    kv_len: torch.Tensor
    state_slots: torch.Tensor
    logit_rows: torch.Tensor
    num_logit_rows: int
    # every request cut into tiles of at most 128 consecutive rows: int32 [num_q_tiles, 4] =
    # (request, first row of the step, rows, first position)
    # The tiles of prompt portions come first (those that read the most keys first), then the one-row tiles of
    # the requests at the head of the step that bring a single token each (`leading_decode_rows` of them, rows
    # 0 .. leading_decode_rows - 1): a mixer may hand those rows to its decode kernel and only the first
    # `num_prompt_q_tiles` tiles to its prompt kernel.
    q_tiles: Optional[torch.Tensor] = None
    num_q_tiles: int = 0
    num_prompt_q_tiles: int = 0
    leading_decode_rows: int = 0
    h_q_len: List[int] = field(default_factory=list)
    h_pos_start: List[int] = field(default_factory=list)
    h_state_slots: List[int] = field(default_factory=list)
    block_tables: Dict[int, torch.Tensor] = field(default_factory=dict)   # cache group -> [requests, max_blocks]
    decode_only: bool = False        # every request brings exactly one token
    max_q_len: int = 0
    max_kv_len: int = 0
    extras: Dict[str, object] = field(default_factory=dict)   # per-step scratch parts may share (launch plans)
