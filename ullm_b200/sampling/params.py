"""Request-level datatypes, with the reference's names and meanings
(ullm/core/common.py:7-43)."""

from __future__ import annotations

import enum
from dataclasses import dataclass, field


@dataclass
class SamplingParams:
    """ullm/core/common.py:7-19.  `max_tokens` bounds the TOTAL length (prompt +
    generated), `max_new_tokens` the generated tokens (ullm/core/engine.py:
    184-194).  temperature <= 0 means greedy argmax here (the reference replaces
    it by 1.0, ullm/layers/sampler.py:41, and reaches greedy only as top_k=1).
    `seed`: this engine's addition; the draw of step n of a request depends only
    on (seed, n), never on what else is in the batch."""

    n: int = 1
    temperature: float = 1.0
    top_p: float = 1.0
    top_k: int = -1
    min_p: float = 0.0
    max_tokens: int | None = None
    max_new_tokens: int | None = None
    stop: list[str] = field(default_factory=list)
    ignore_eos: bool = False
    eos_token_id: int = -1
    seed: int | None = None


class FinishReason(enum.Enum):
    STOP = enum.auto()
    LENGTH = enum.auto()
    ABORT = enum.auto()


@dataclass
class GenerateOutput:
    """One streamed token (ullm/core/common.py:27-33) plus its id."""

    token_str: str
    is_finished: bool
    finish_reason: FinishReason | None
    num_prompt_tokens: int
    num_generated_tokens: int
    token_id: int = -1


class EngineDeadError(Exception):
    """Raised by the entry point's calls once a step of the engine has failed (ullm/core/common.py:46-54: there
    the engine is a process that has exited; here it lives in this process and is not stepped again after a
    step raised, since the cache and the requests in flight are in an unknown state)."""

    MESSAGE = "The engine has failed and takes no more requests."

    def __init__(self, message: str = MESSAGE, *args):
        super().__init__(message, *args)


@dataclass
class EngineStepResult:
    """ullm/core/common.py:36-43."""

    seq_id: str
    new_token_id: int
    is_finished: bool
    finish_reason: FinishReason | None
    num_prompt_tokens: int
    num_generated_tokens: int


@dataclass
class RequestOutput:
    """A finished request of the synchronous entry point."""

    request_id: str
    prompt_token_ids: list[int]
    token_ids: list[int]
    finish_reason: FinishReason | None
    text: str | None = None

    @property
    def num_prompt_tokens(self) -> int:
        return len(self.prompt_token_ids)

    @property
    def num_generated_tokens(self) -> int:
        return len(self.token_ids)
