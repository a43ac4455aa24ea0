"""ullm_b200: a single-GPU (B200, sm_100a) inference engine for the Qwen3 dense
decoder, built from exchangeable parts."""

__version__ = "0.1.0"


def __getattr__(name):
    # The public names of the reference (ullm/__init__.py:10-17), loaded on demand so
    # that importing the package for its config or weights tools stays light.
    if name in ("LLM", "RequestOutput"):
        from .engine import llm

        return getattr(llm, name)
    if name == "EngineConfig":
        from .config import EngineConfig

        return EngineConfig
    if name in ("SamplingParams", "FinishReason", "GenerateOutput", "EngineDeadError"):
        from .sampling import params

        return getattr(params, name)
    raise AttributeError(name)
