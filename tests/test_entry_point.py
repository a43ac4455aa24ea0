"""The Python entry point's behaviour that needs no GPU: what happens after a step of the engine has failed."""

import asyncio
from types import SimpleNamespace

import pytest

import ullm_b200
from ullm_b200.engine.llm import LLM
from ullm_b200.sampling.params import EngineStepResult, SamplingParams


class _FailingEngine:
    """Stands in for the engine: hands out one token, then its step raises."""

    context_len = 64

    def __init__(self):
        from types import SimpleNamespace

        self.runner = SimpleNamespace(spec=SimpleNamespace(eos_token_id=None))
        self.live: list[str] = []
        self.steps = 0
        self.profile_steps = False

    def add_sequence(self, sid, ids, params):
        self.live.append(sid)

    def abort_sequence(self, sid):
        self.live.remove(sid)

    def has_unfinished_sequences(self):
        return bool(self.live)

    def step(self):
        self.steps += 1
        if self.steps > 1:
            raise RuntimeError("kernel status 6")
        return [EngineStepResult(s, 7, False, None, 0, 0) for s in self.live]

    def shutdown(self):
        pass


def _llm() -> LLM:
    llm = LLM.__new__(LLM)
    llm.config = SimpleNamespace(get_default_sampling_params=SamplingParams)
    llm.engine = _FailingEngine()
    llm.tokenizer = None
    llm.request_states = {}
    llm._loop_task = None
    llm.is_dead = False
    return llm


def test_exports_follow_the_reference():
    """ullm/__init__.py:10-17."""
    for name in ("LLM", "EngineConfig", "SamplingParams", "FinishReason", "GenerateOutput", "EngineDeadError"):
        assert getattr(ullm_b200, name) is not None


def test_a_failed_step_reaches_the_caller_and_the_engine_takes_no_more_requests():
    llm = _llm()
    with pytest.raises(RuntimeError, match="kernel status 6"):
        llm.generate_batch([[1, 2, 3]], SamplingParams(max_new_tokens=4))
    assert llm.is_dead and llm.engine.steps == 2
    with pytest.raises(ullm_b200.EngineDeadError):
        llm.generate_batch([[1, 2, 3]], SamplingParams(max_new_tokens=4))
    assert llm.engine.steps == 2  # not stepped again


def test_streaming_generators_get_the_failure_and_later_calls_raise_engine_dead():
    llm = _llm()

    async def run():
        got = []
        with pytest.raises(RuntimeError, match="kernel status 6"):
            async for out in llm.generate([1, 2, 3], SamplingParams(max_new_tokens=4), "a"):
                got.append(out.token_id)
        assert got == [7]
        with pytest.raises(ullm_b200.EngineDeadError):
            async for _ in llm.generate([1, 2], None, "b"):
                pass
        with pytest.raises(ullm_b200.EngineDeadError):
            await llm.profile("start")
        llm.abort("a")  # harmless on a dead engine
        await llm.shutdown()

    asyncio.run(run())
