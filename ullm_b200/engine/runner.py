"""The step function: runs a batch of (request, its next tokens) through the
model from the cache and returns the logits at the wanted places.

ullm/core/model_runner.py:298-363 is the reference's `execute_model`; it takes
either whole uncached prompts or single decode tokens, never both.  Here a
step holds any mix: portions of prompts of any length beside single decoded
tokens, and the logits rows are chosen by the caller.

The runner owns the model, the cache manager, the step's staging buffers and
the activation workspace.  It decides nothing about which requests run: the
scheduler (engine.scheduler) or a replayed trace (bin/trace_run) does.
"""

from __future__ import annotations

import logging

import numpy as np
import torch

from ..cache import CacheManager, OutOfPages, RequestCache
from ..config.registry import load_model_spec
from ..csrc import kernels
from ..parts.model import DecoderModel
from ..weights import files_have, fill_random_, load_weights
from .batch import GroupStep, StepContext, StepEntry, StepStaging, Workspace

logger = logging.getLogger("ullm_b200")

_TORCH_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


def engine_dtype(requested: str | None, checkpoint: str) -> torch.dtype:
    """The compute dtype: the caller's choice, else the checkpoint's (ullm/core/model_runner.py:38-51 takes
    config.json's).  float16 is served in float16: weights, cache and activations are float16, the arithmetic
    inside the kernels is 32-bit as in the other two; its attention runs on the plain kernel (the tensor-core
    attention kernels take bfloat16 only), so it is the slow one of the two 16-bit types."""
    name = requested or checkpoint
    name = {"bf16": "bfloat16", "fp32": "float32", "fp16": "float16", "half": "float16"}.get(name, name)
    if name not in _TORCH_DTYPES:
        raise ValueError(f"Unsupported dtype {name!r}")
    return _TORCH_DTYPES[name]


class ModelRunner:
    def __init__(
        self,
        model_dir: str | None = None,
        *,
        config: dict | None = None,
        dtype: str | None = None,
        device: str = "cuda:0",
        page_size: int = 16,
        num_pages: int | None = None,
        gpu_memory_utilization: float = 0.9,
        max_requests: int = 8,
        max_context: int = 2048,
        max_step_tokens: int = 2048,
        load_format: str = "safetensors",
        seed: int = 0,
        random_std: float = 0.02,
        random_norm_std: float = 0.0,
        enable_prefix_cache: bool = False,
        poison_cache: bool = False,
        progress=None,
    ):
        if model_dir is None and config is None:
            raise ValueError("a model folder or a config dict is needed")
        self.device = torch.device(device)
        self.typed_config, self.spec = load_model_spec(config if config is not None else model_dir)
        self.dtype = engine_dtype(dtype, self.spec.dtype)
        self.checkpoint_dtype = self.spec.dtype
        if self.dtype == torch.float16:
            logger.warning("serving in float16 (%s): correct, but attention runs on the plain kernel; the tensor-core "
                           "attention kernels take bfloat16 (dtype='bfloat16' selects them)",
                           "asked for" if dtype else "config.json's dtype, or its default when the key is absent")
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
            # a true 32-bit path: no reduced-precision matrix mode, ever
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
            torch.set_float32_matmul_precision("highest")
        untie = False
        if load_format == "safetensors" and self.spec.tie_embeddings:
            untie = files_have(model_dir, self.spec.head_name + "weight")
        self.model = DecoderModel(self.spec, untie_head=untie)
        self.model.allocate(self.device, self.dtype)
        if load_format == "safetensors":
            if model_dir is None:
                raise ValueError("load_format='safetensors' needs a model folder")
            load_weights(self.model, model_dir, progress)
        elif load_format == "random":
            fill_random_(self.model, seed, random_std, random_norm_std)
        else:
            raise ValueError(f"unknown load_format {load_format!r}")

        self.page_size = page_size
        self.max_context = min(max_context, self.spec.max_positions)
        self.max_requests = max_requests
        self.max_step_tokens = max_step_tokens
        needs = self.model.cache_needs()
        pages_per_request = -(-self.max_context // page_size)
        if num_pages is None:
            num_pages = self._pages_from_memory(needs, gpu_memory_utilization, pages_per_request)
        self.cache = CacheManager(
            needs, page_size, num_pages, max_requests, pages_per_request, device=self.device, dtype=self.dtype,
            enable_prefix_cache=enable_prefix_cache, poison=poison_cache,
        )
        self.staging = StepStaging(self.device, max_step_tokens, max_requests, len(self.cache.groups))
        # decode steps have few integers: a small buffer of their own keeps their copy small
        self.decode_staging = StepStaging(self.device, max_requests, max_requests, len(self.cache.groups))
        self.workspace = Workspace(self.device, max_tokens=max_step_tokens, max_requests=max_requests)
        # per-request state of fixed size: the token each request sampled last, by request slot
        self.last_tokens = torch.zeros(max_requests, dtype=torch.int32, device=self.device)
        self.steps_run = 0
        self._staged = torch.cuda.Event() if self.device.type == "cuda" else None

    # -- sizing ----------------------------------------------------------------
    def _pages_from_memory(self, needs, utilization: float, pages_per_request: int) -> int:
        """ullm/core/model_runner.py:233-255 sizes the pool from the memory that
        is free once the weights are resident, times gpu_memory_utilization.
        Room for one step's activations is set aside first."""
        itemsize = torch.empty((), dtype=self.dtype).element_size()
        per_page = CacheManager.bytes_per_page(needs, self.page_size, itemsize)
        if self.device.type != "cuda":
            return max(1, self.max_requests * pages_per_request)
        free, _total = torch.cuda.mem_get_info(self.device)
        reserve = self._activation_bytes()
        budget = int(free * utilization) - reserve
        pages = budget // max(per_page, 1)
        cap = self.max_requests * pages_per_request * 2
        pages = min(pages, cap)
        if pages < pages_per_request:
            raise RuntimeError(
                f"not enough device memory for one request of {self.max_context} tokens: "
                f"{pages} pages fit, {pages_per_request} needed")
        return int(pages)

    def _activation_bytes(self) -> int:
        """Room for one step's work buffers: every part says how many elements per token it keeps in the
        workspace (`Part.activation_elems`); layers reuse the buffers, so the widest layer counts."""
        s = self.spec
        widest = max((b.activation_elems() for b in self.model.blocks), default=0)
        itemsize = torch.empty((), dtype=self.dtype).element_size()
        acts = self.max_step_tokens * (widest + 2 * s.hidden_size) * itemsize
        logits = self.max_requests * s.vocab_size * 4 * 2
        return int(acts + logits + (512 << 20))

    # -- requests -----------------------------------------------------------------
    def add_request(self, request_id: str, tokens=None) -> RequestCache | None:
        return self.cache.admit(request_id, tokens)

    def end_request(self, request_id: str, tokens=None) -> None:
        self.cache.release(self.cache.requests[request_id], tokens)

    def has_request(self, request_id: str) -> bool:
        return request_id in self.cache.requests

    # -- the step -------------------------------------------------------------------
    def prepare(self, entries: list[StepEntry], pad_to: int | None = None, staging=None) -> StepContext:
        """Reserves pages for the step's tokens and stages its integers on the
        device.  Raises OutOfPages (nothing of the step has run then; pages
        reserved for earlier entries stay with their requests).

        `pad_to` (decode steps replayed from a CUDA graph): the batch is filled
        up to that many one-token rows that belong to no request: token 0,
        batch row -1 (attention writes zeros), slot -1 (nothing is stored); their
        logits rows are computed and ignored."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        cache = self.cache
        B = len(entries)
        T = sum(len(e.tokens) for e in entries)
        R = sum(len(e.want) for e in entries)
        V = self.spec.vocab_size
        rcs = []
        seen = set()
        orig_entries = entries
        for e in list(entries):
            if e.request_id in seen:
                raise ValueError(f"request {e.request_id!r} appears twice in one step")
            seen.add(e.request_id)
            rc = cache.requests.get(e.request_id)
            if rc is None:
                raise KeyError(f"request {e.request_id!r} is not live (add_request first)")
            n = len(e.tokens)
            if n == 0:
                raise ValueError(f"request {e.request_id!r}: a step entry needs at least one token")
            if rc.num_tokens + n > self.max_context:
                raise ValueError(
                    f"request {e.request_id!r}: {rc.num_tokens} + {n} tokens exceed the context of {self.max_context}")
            if n == 1 and e.tokens[0] == -1:
                pass  # "the token this request sampled last": resolved on the device
            elif n <= 16:
                if min(e.tokens) < 0 or max(e.tokens) >= V:
                    bad = [t for t in e.tokens if not 0 <= t < V]
                    raise ValueError(f"request {e.request_id!r}: token id {bad[0]} is outside the vocabulary of {V}")
            else:
                arr = np.asarray(e.tokens, dtype=np.int64)
                if int(arr.min()) < 0 or int(arr.max()) >= V:
                    bad = arr[(arr < 0) | (arr >= V)]
                    raise ValueError(
                        f"request {e.request_id!r}: token id {int(bad[0])} is outside the vocabulary of {V}")
                e = StepEntry(e.request_id, arr, e.want)  # the array is what gets copied below
                entries = entries if entries is not orig_entries else list(orig_entries)
                entries[len(rcs)] = e
            badw = [w for w in e.want if not 0 <= w < n]
            if badw:
                raise ValueError(f"request {e.request_id!r}: wanted place {badw[0]} is outside its {n} tokens")
            rcs.append(rc)
        for e, rc in zip(entries, rcs):
            cache.reserve(rc, len(e.tokens))

        st = staging if staging is not None else self.staging
        st.ensure(max(T, pad_to or 0), max(B, pad_to or 0))
        lay = st.layout(st.max_tokens, st.max_requests)
        if self._staged is not None:
            self._staged.synchronize()  # the previous step's copy out of the pinned buffer is done
        h = st.host.numpy()

        def seg(name):
            off, _n = lay[name]
            return off

        o_ids, o_pos, o_req, o_rows = seg("token_ids"), seg("positions"), seg("token_req"), seg("logits_rows")
        o_cu, o_kv, o_rs = seg("cu_q"), seg("kv_len"), seg("req_slots")
        t = 0
        r = 0
        cu = [0]
        starts = []
        max_q = max_kv = 1
        sum_kv = 0
        one_token_each = T == B
        if one_token_each:
            # a decode step: every segment is filled by one assignment instead of one per entry
            ps = cache.page_size
            starts = [rc.num_tokens for rc in rcs]
            h[o_ids:o_ids + B] = [e.tokens[0] for e in entries]
            h[o_pos:o_pos + B] = starts
            h[o_req:o_req + B] = range(B)
            for g in range(len(cache.groups)):
                o_sm = seg(f"slot_mapping{g}")
                h[o_sm:o_sm + B] = [rc.pages[g][s // ps] * ps + s % ps for rc, s in zip(rcs, starts)]
            rows = [b for b, e in enumerate(entries) for _ in e.want]
            h[o_rows:o_rows + len(rows)] = rows
            h[o_kv:o_kv + B] = [s + 1 for s in starts]
            h[o_rs:o_rs + B] = [rc.slot for rc in rcs]
            t, r = B, len(rows)
            cu = list(range(B + 1))
            max_kv = max(starts) + 1
            sum_kv = sum(starts) + B
        for b, (e, rc) in enumerate(() if one_token_each else zip(entries, rcs)):
            n = len(e.tokens)
            start = rc.num_tokens
            starts.append(start)
            h[o_ids + t:o_ids + t + n] = e.tokens
            h[o_pos + t:o_pos + t + n] = np.arange(start, start + n, dtype=np.int32) if n > 16 else range(start, start + n)
            h[o_req + t:o_req + t + n] = b
            for g in range(len(cache.groups)):
                o_sm = seg(f"slot_mapping{g}")
                h[o_sm + t:o_sm + t + n] = cache.slot_mapping(rc, g, n)
            for w in e.want:
                h[o_rows + r] = t + w
                r += 1
            h[o_kv + b] = start + n
            h[o_rs + b] = rc.slot
            t += n
            cu.append(t)
            max_q = max(max_q, n)
            max_kv = max(max_kv, start + n)
            sum_kv += start + n
        if pad_to is not None and pad_to > B:
            if T != B:
                raise ValueError("only one-token steps can be padded")
            extra = pad_to - B
            h[o_ids + t:o_ids + t + extra] = 0
            h[o_pos + t:o_pos + t + extra] = 0
            h[o_req + t:o_req + t + extra] = -1
            for g in range(len(cache.groups)):
                o_sm = seg(f"slot_mapping{g}")
                h[o_sm + t:o_sm + t + extra] = -1
            h[o_rows + r:o_rows + r + extra] = range(t, t + extra)
            h[o_kv + B:o_kv + pad_to] = 0
            h[o_rs + B:o_rs + pad_to] = 0
            cu.extend(range(t + 1, t + extra + 1))
            T = R = B = pad_to
        h[o_cu:o_cu + B + 1] = cu
        cache.flush_block_tables()
        end = lay["_end"][0]
        st.dev[:end].copy_(st.host[:end], non_blocking=True)
        if self._staged is not None:
            self._staged.record()

        d = st.dev
        kv_len = d[o_kv:o_kv + B]
        req_slots = d[o_rs:o_rs + B]
        groups = []
        for g, info in enumerate(cache.groups):
            o_sm = seg(f"slot_mapping{g}")
            groups.append(GroupStep(cache.block_tables[g], kv_len, d[o_sm:o_sm + T], req_slots,
                                    cache.page_size, info.need.window))
        return StepContext(
            num_tokens=T, num_requests=B, num_logits_rows=R,
            token_ids=d[o_ids:o_ids + T], positions=d[o_pos:o_pos + T], token_req=d[o_req:o_req + T],
            cu_q=d[o_cu:o_cu + B + 1], logits_rows=d[o_rows:o_rows + R], req_slots=req_slots,
            groups=groups, workspace=self.workspace,
            cu_q_host=cu, req_slots_host=[rc.slot for rc in rcs] + [0] * (B - len(rcs)),
            start_positions_host=starts + [0] * (B - len(rcs)),
            max_q_len=max_q, max_kv_len=max_kv, decode_only=(max_q == 1), last_tokens=self.last_tokens,
            sum_kv_len=sum_kv, num_live_requests=len(entries),
        )

    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Runs the entries as one batch.  Returns the logits at the wanted
        places, float32 [wanted, vocab] in the order of the entries and of their
        `want` lists (a view of a buffer that the next step overwrites), or None
        when nothing is wanted."""
        ctx = self.prepare(entries)
        logits = self.run_model(ctx)
        self.commit(entries)
        return logits

    def run_model(self, ctx: StepContext) -> torch.Tensor | None:
        if self.device.type == "cuda":
            kernels().begin_step(ctx.num_tokens, self.dtype)  # (kernel choices that go by the size of the step)
        return self.model.forward(ctx, self.cache.layer_caches(ctx.groups))

    def commit(self, entries: list[StepEntry]) -> None:
        for e in entries:
            self.cache.commit(self.cache.requests[e.request_id], len(e.tokens))
        self.steps_run += 1

    def check_device_status(self) -> None:
        if self.device.type == "cuda":
            kernels().raise_on_status()
