"""The flat batch of one step and the buffers it lives in.

The reference rebuilds flat arrays per step in `InputBatch.update_batch`
(ullm/core/input_batch.py:80-220): ids, positions, the slots new keys go to,
cumulative lengths, the rows whose logits are wanted.  Here a step's integer
inputs are packed into ONE pinned host buffer and reach the device in one
copy; the block tables are already there (the cache manager keeps them).
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens (a prompt portion, or one
    decoded token) and the places among them whose logits are wanted."""

    request_id: str
    tokens: list[int]
    want: list[int] = field(default_factory=list)


@dataclass
class GroupStep:
    """A cache group's metadata for this step (device tensors)."""

    block_table: torch.Tensor  # [slots, pages per request] int32, indexed by request slot
    kv_len: torch.Tensor  # [B] int32: tokens each request holds after this step
    slot_mapping: torch.Tensor  # [T] int32: flat slot of each new token (-1: none)
    req_slots: torch.Tensor  # [B] int32: request slot of each batch row
    page_size: int
    window: int | None


class Workspace:
    """Named activation buffers that persist across steps (so a captured CUDA
    graph finds them at the same address).  A buffer is known by (name, columns,
    dtype): two layers of different width that use the same name get a buffer
    each, so a model whose layers differ neither reallocates per layer nor
    invalidates recorded graphs.  `get` returns the first `rows` rows; a buffer
    grows when more rows are asked for than it has, which bumps `generation`
    (anything that recorded addresses must be re-recorded).  To keep that rare,
    a buffer is made at once for what its caller says it may ever need
    (`reserve` rows): per-token buffers for the largest step (`max_tokens`),
    per-request buffers for all request slots (`max_requests`)."""

    def __init__(self, device, max_tokens: int = 0, max_requests: int = 0):
        self.device = device
        self.max_tokens = max_tokens
        self.max_requests = max_requests
        self.buffers: dict[tuple, torch.Tensor] = {}
        self.generation = 0

    def get(self, name: str, rows: int, cols: int, dtype: torch.dtype, reserve: int = 0) -> torch.Tensor:
        key = (name, cols, dtype)
        buf = self.buffers.get(key)
        if buf is None or buf.shape[0] < rows:
            cap = max(rows, reserve, 0 if buf is None else buf.shape[0], 1)
            buf = torch.empty((cap, cols), dtype=dtype, device=self.device)
            self.buffers[key] = buf
            self.generation += 1
        return buf[:rows]

    def tokens(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """A buffer with a row per token of the step."""
        return self.get(name, rows, cols, dtype, reserve=self.max_tokens)

    def requests(self, name: str, rows: int, cols: int, dtype: torch.dtype) -> torch.Tensor:
        """A buffer with a row per request of the step (more rows when a caller wants logits at many places)."""
        return self.get(name, rows, cols, dtype, reserve=self.max_requests)


@dataclass
class StepContext:
    """Everything a part may read about the step.  Device tensors are views of
    the staging buffer; the host lists mirror them for parts that loop on the
    host (a test's toy mixer does)."""

    num_tokens: int
    num_requests: int
    num_logits_rows: int
    token_ids: torch.Tensor  # [T] int32
    positions: torch.Tensor  # [T] int32
    token_req: torch.Tensor  # [T] int32: batch row of each token
    cu_q: torch.Tensor  # [B+1] int32
    logits_rows: torch.Tensor  # [R] int32: flat token rows whose logits are wanted
    req_slots: torch.Tensor  # [B] int32
    groups: list[GroupStep]
    workspace: Workspace
    # host mirrors
    cu_q_host: list[int]
    req_slots_host: list[int]
    start_positions_host: list[int]  # tokens each request held before this step
    max_q_len: int = 1
    max_kv_len: int = 1
    decode_only: bool = False
    last_tokens: torch.Tensor | None = None  # int32 [request slots]: what each request sampled last (for id -1)
    # what a block prepared for the next block's first norm (norm object, operand r * w, sums of squares, eps)
    folded_norm: object = None
    sum_kv_len: int = 0  # tokens all requests of the step hold after it, padding rows not counted
    num_live_requests: int = 0  # requests of the step without padding rows


class StepStaging:
    """Pinned host buffer + device buffer for a step's integers."""

    def __init__(self, device, max_tokens: int, max_requests: int, num_groups: int):
        self.device = torch.device(device)
        self.max_tokens = max_tokens
        self.max_requests = max_requests
        self.num_groups = num_groups
        n = self.size_for(max_tokens, max_requests)
        pin = self.device.type == "cuda"
        self.host = torch.zeros(n, dtype=torch.int32, pin_memory=pin)
        self.dev = torch.zeros(n, dtype=torch.int32, device=self.device)

    def size_for(self, T: int, B: int) -> int:
        # ids, positions, token_req, logits_rows, slot_mapping per group: T each;
        # cu_q: B+1; kv_len, req_slots: B each.  Segments start on 4-int boundaries.
        def up(x):
            return (x + 3) // 4 * 4

        return up(T) * (4 + self.num_groups) + up(B + 1) + 2 * up(B)

    def ensure(self, T: int, B: int) -> None:
        if T > self.max_tokens or B > self.max_requests:
            self.max_tokens = max(T, self.max_tokens)
            self.max_requests = max(B, self.max_requests)
            n = self.size_for(self.max_tokens, self.max_requests)
            pin = self.device.type == "cuda"
            self.host = torch.zeros(n, dtype=torch.int32, pin_memory=pin)
            self.dev = torch.zeros(n, dtype=torch.int32, device=self.device)

    def layout(self, T: int, B: int) -> dict[str, tuple[int, int]]:
        """Offsets for capacities (T, B): segments are laid out for the CAPACITY
        so that a fixed capacity gives fixed addresses."""

        def up(x):
            return (x + 3) // 4 * 4

        off, out = 0, {}
        for name in ("token_ids", "positions", "token_req", "logits_rows"):
            out[name] = (off, T)
            off += up(T)
        for g in range(self.num_groups):
            out[f"slot_mapping{g}"] = (off, T)
            off += up(T)
        out["cu_q"] = (off, B + 1)
        off += up(B + 1)
        out["kv_len"] = (off, B)
        off += up(B)
        out["req_slots"] = (off, B)
        off += up(B)
        out["_end"] = (off, 0)
        return out
