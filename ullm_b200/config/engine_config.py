"""EngineConfig: the options of one engine instance.

Names and meanings follow ullm/config.py:9-25 (`model`,
`gpu_memory_utilization`, `max_bs`, `tp_size`, `pp_size`, `nccl_port`,
`device_ids`, `enforce_eager`, `context_len`, `disable_async_scheduling`,
`log_level`, `profile`, `profile_dir`) and its `from_args` (:69-88).  This
engine runs on one GPU in one process: tp_size and pp_size are accepted and
must be 1, nccl_port is accepted and unused.  Added here: the page size, the
token budget of a step, the compute dtype, the way weights come to be, a seed,
and an explicit page count for tests.
"""

from __future__ import annotations

import argparse
import json
import os
from dataclasses import dataclass, field
from typing import Any


@dataclass
class EngineConfig:
    model: str
    gpu_memory_utilization: float = 0.9
    max_bs: int = 50
    tp_size: int = 1
    pp_size: int = 1
    nccl_port: int = 29500
    device_ids: list[int] | None = None
    enforce_eager: bool = False
    context_len: int = 2048
    disable_async_scheduling: bool = False
    log_level: str = "info"
    profile: bool = False
    profile_dir: str = "./profiles"

    # additions of this engine
    page_size: int = 16
    max_num_batched_tokens: int = 2048
    dtype: str | None = None  # None: config.json's; "bfloat16" | "float32"
    load_format: str = "safetensors"  # "safetensors" | "random" (seeded, made on the device)
    seed: int = 0
    num_pages: int | None = None  # None: sized from free memory x gpu_memory_utilization
    enable_prefix_caching: bool = True
    warmup_graphs: bool = False  # record every decode graph while the engine starts instead of at first use
    random_init_std: float = 0.02
    random_init_norm_std: float = 0.0

    model_config: dict[str, Any] = field(init=False, repr=False)
    generation_config: dict[str, Any] | None = field(init=False, repr=False)

    def __post_init__(self):
        if self.tp_size != 1 or self.pp_size != 1:
            raise ValueError("this engine runs on one GPU: tp_size and pp_size must be 1")
        if self.device_ids is not None and len(self.device_ids) != 1:
            raise ValueError("this engine runs on one GPU: device_ids must name one device")
        if not 0.0 < self.gpu_memory_utilization <= 1.0:
            raise ValueError("gpu_memory_utilization must be in (0, 1]")
        if self.max_bs <= 0 or self.context_len <= 0 or self.page_size <= 0:
            raise ValueError("max_bs, context_len and page_size must be positive")
        if self.max_num_batched_tokens <= 0:
            raise ValueError("max_num_batched_tokens must be positive")
        if self.dtype is not None:
            self.dtype = {"bf16": "bfloat16", "fp32": "float32", "fp16": "float16", "half": "float16"}.get(
                self.dtype, self.dtype)
            if self.dtype not in ("bfloat16", "float32", "float16"):
                raise ValueError(f"Unsupported dtype {self.dtype!r} (bfloat16, float16 or float32)")
        if self.load_format not in ("safetensors", "random"):
            raise ValueError("load_format is 'safetensors' or 'random'")
        from .registry import read_config_json

        self.model_config = read_config_json(self.model)
        gpath = os.path.join(self.model, "generation_config.json")
        self.generation_config = None
        if os.path.isfile(gpath):
            with open(gpath) as f:
                self.generation_config = json.load(f)

    def get_default_sampling_params(self):
        """ullm/config.py:46-67: temperature, top_k, top_p and min_p of
        generation_config.json override the defaults of SamplingParams."""
        from ..sampling.params import SamplingParams

        if not self.generation_config:
            return SamplingParams()
        kw = {k: self.generation_config[k] for k in ("temperature", "top_k", "top_p", "min_p")
              if self.generation_config.get(k) is not None}
        return SamplingParams(**kw)

    @property
    def device(self) -> str:
        return f"cuda:{self.device_ids[0]}" if self.device_ids else "cuda:0"

    @staticmethod
    def add_cli_args(parser: argparse.ArgumentParser) -> None:
        """The reference's flags (ullm/entrypoints/api_server.py:127-184) with
        its defaults, then this engine's own."""
        parser.add_argument("--model", type=str, required=True, help="Model folder (config.json + *.safetensors)")
        parser.add_argument("--gpu-memory-utilization", type=float, default=0.9, help="GPU memory utilization")
        parser.add_argument("--max-bs", type=int, default=50, help="Maximum batch size")
        parser.add_argument("--tp-size", type=int, default=1, help="Tensor parallel size (must be 1)")
        parser.add_argument("--pp-size", type=int, default=1, help="Pipeline parallel size (must be 1)")
        parser.add_argument("--nccl-port", type=int, default=29500, help="Accepted for compatibility; unused")
        parser.add_argument("--device-ids", type=str, default=None, help="GPU device id to use")
        parser.add_argument("--context-len", type=int, default=2048, help="Max context length of the model")
        parser.add_argument("--enforce-eager", action="store_true", help="Enforce eager execution, disable CUDA graph")
        parser.add_argument("--log-level", type=str, default="info", help="Log level for the engine")
        parser.add_argument("--profile", action="store_true", help="Time every step (and the kernel groups of eager steps); printed and written to --profile-dir at the end")
        parser.add_argument("--profile-dir", type=str, default="./profiles", help="Directory to save profiling results")
        parser.add_argument("--disable-async-scheduling", action="store_true",
                            help="Disable asynchronous scheduling (read every step before launching the next)")
        parser.add_argument("--page-size", type=int, default=16, help="Tokens per KV page")
        parser.add_argument("--max-num-batched-tokens", type=int, default=2048, help="Token budget of one step")
        parser.add_argument("--dtype", type=str, default=None, help="bfloat16, float16 or float32 (default: config.json's; the fast attention kernels are bfloat16)")
        parser.add_argument("--load-format", type=str, default="safetensors", help="safetensors or random")
        parser.add_argument("--seed", type=int, default=0, help="Seed of random weights and of sampling")
        parser.add_argument("--num-pages", type=int, default=None, help="KV pages (default: from free memory)")
        parser.add_argument("--no-prefix-caching", action="store_true", help="Disable prefix reuse over pages")
        parser.add_argument("--warmup-graphs", action="store_true",
                            help="Record the CUDA graphs of all decode batch sizes at start-up (default: at first use)")

    @staticmethod
    def from_args(args: argparse.Namespace) -> "EngineConfig":
        device_ids = [int(i) for i in args.device_ids.split(",")] if args.device_ids else None
        return EngineConfig(
            model=args.model,
            gpu_memory_utilization=args.gpu_memory_utilization,
            max_bs=args.max_bs,
            tp_size=args.tp_size,
            pp_size=args.pp_size,
            nccl_port=args.nccl_port,
            device_ids=device_ids,
            enforce_eager=args.enforce_eager,
            context_len=args.context_len,
            log_level=args.log_level,
            profile=args.profile,
            profile_dir=args.profile_dir,
            disable_async_scheduling=args.disable_async_scheduling,
            page_size=getattr(args, "page_size", 16),
            max_num_batched_tokens=getattr(args, "max_num_batched_tokens", 2048),
            dtype=getattr(args, "dtype", None),
            load_format=getattr(args, "load_format", "safetensors"),
            seed=getattr(args, "seed", 0),
            num_pages=getattr(args, "num_pages", None),
            enable_prefix_caching=not getattr(args, "no_prefix_caching", False),
            warmup_graphs=getattr(args, "warmup_graphs", False),
        )
