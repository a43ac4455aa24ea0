"""Python face of the compiled kernels: loads the shared library with ctypes
and wraps each extern "C" launcher in a method that checks devices, dtypes,
shapes and contiguity before passing raw pointers and the current CUDA stream.

There is no CPU path here: a tensor that is not on a CUDA device is an error,
and a missing or unbuildable library is an error at first use.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .build import build

_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_ERRORS = {
    1: "unsupported dtype",
    2: "bad size argument",
    3: "CUDA launch failed",
    4: "size not supported by this kernel",
}
STATUS_MESSAGES = {
    1: "token id out of range (row {index}: id {value})",
    2: "position out of range of the position table (token {index}: position {value})",
    3: "cache slot out of range (token {index}: slot {value})",
    4: "row index out of range (row {index}: {value})",
    5: "page id out of range in a block table (token {index}: page {value})",
    6: "a kernel gave up waiting on a barrier (place {index}, at {value}) and returned early",
}

MAX_HEAD_DIM = 512


class KernelError(RuntimeError):
    pass


def check_attention_sizes(num_heads: int, num_kv_heads: int, head_dim: int, rotary_dim: int) -> None:
    """Sizes the attention kernels take; anything else is refused here, at
    construction, with the reason."""
    if num_heads <= 0 or num_kv_heads <= 0 or num_heads % num_kv_heads:
        raise ValueError(f"num_heads={num_heads} must be a positive multiple of num_kv_heads={num_kv_heads}")
    if head_dim <= 0 or head_dim > MAX_HEAD_DIM:
        raise ValueError(f"head_dim={head_dim}: the attention kernels take 1..{MAX_HEAD_DIM}")
    if rotary_dim < 0 or rotary_dim > head_dim or rotary_dim % 2:
        raise ValueError(f"rotary_dim={rotary_dim} must be even and at most head_dim={head_dim}")


def _ptr(t: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if t is None else t.data_ptr())


def _stream() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}: the kernels run on CUDA tensors only (no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _timed(group: str, nbytes=None, skipped=None):
    """While a timer is installed (`Kernels.timer`, see engine/profiler.py), the wrapped call is bracketed by
    two CUDA events and booked under `group`; `nbytes(*args)` says what it had to read, if that is known.
    `skipped`: what the call returns when a measurement leaves its group out."""

    def outer(fn):
        def inner(self, *a, **k):
            if self.skip_groups and group in self.skip_groups:
                return skipped  # a measurement leaves this group out (the step's results are then meaningless)
            t = self.timer
            if t is None:
                return fn(self, *a, **k)
            start = t.begin()
            try:
                return fn(self, *a, **k)
            finally:
                t.end(group, start, nbytes(*a) if (nbytes is not None and start is not None) else 0)

        inner.__name__, inner.__doc__ = fn.__name__, fn.__doc__
        return inner

    return outer


def _weight_bytes(x, weight, *rest):
    return weight.numel() * weight.element_size()


class Kernels:
    def __init__(self, lib_path: str | None = None):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device: this engine has no CPU path")
        self.lib_path = lib_path or build()
        self.lib = ctypes.CDLL(self.lib_path)
        self._declare()
        self.status = torch.zeros(4, dtype=torch.int32, device="cuda")
        self.sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
        self._f32_out_mm = None
        self._lin_ws = None  # partial sums and tile counters of the tcgen05 product, made at its first use
        self._lin_counters = None
        self.pdl = False
        self._decb = {}  # (head_dim, heads per kv head) -> (partials, prefix) of the balanced decode attention
        self._tail_ws = {}  # hidden size -> (scratch, counters) of the fused layer tail
        self.apply_switches(os.environ)
        self._lt_ok = None
        self._lt_ws = None
        self._lt_tuned = set()
        self.timer = None  # a KernelGroupTimer while a profile is being taken
        # groups of kernels (the names `_timed` books them under) that are NOT launched: only for measuring what a
        # group costs inside a step, by the difference; the step's results are wrong while this is set
        self.skip_groups: frozenset = frozenset()
        self.attention_path = None  # which attention kernel the last call chose (tests read it)
        self.launches = 0  # hand-written kernels launched (graph replays add what they captured)

    def begin_step(self, rows: int, dtype) -> None:
        """Called by the step function before a step's kernels are launched (or recorded into a CUDA graph): with
        the automatic policy, programmatic dependent launch is on for exactly the steps whose products are all the
        stream kernel (bfloat16, at most `stream_all_rows` rows), and off otherwise."""
        if self.pdl_mode == "auto":
            self.set_pdl(bool(dtype == torch.bfloat16 and self.small_m_mode == "auto" and rows <= self.stream_all_rows))

    # -- switches -----------------------------------------------------------
    SWITCHES = ("ULLM_B200_PDL", "ULLM_B200_DECODE_SPLIT_TARGET", "ULLM_B200_TC_ATTN", "ULLM_B200_DECODE_CLUSTER",
                "ULLM_B200_FUSE_DECODE_ROPE", "ULLM_B200_MIXED_DECODE_ROWS", "ULLM_B200_DECODE_TC",
                "ULLM_B200_DECODE_BALANCED", "ULLM_B200_SMALL_M_LINEAR", "ULLM_B200_STREAM_WEIGHT_MB",
                "ULLM_B200_FUSED_MLP_ROWS", "ULLM_B200_LT_ROWS", "ULLM_B200_FUSED_TAIL_ROWS",
                "ULLM_B200_STREAM_ALL_ROWS", "ULLM_B200_CHAIN_NORMS")

    def apply_switches(self, env) -> None:
        """Sets every kernel choice from `env` (a mapping; the process environment at start-up): a switch that is
        not in it takes its default.  All switches are optional; the defaults are what was measured fastest."""
        get = env.get
        # programmatic dependent launch for every kernel of the library: "auto" (the default) for the steps whose
        # products are all the stream kernel (see `begin_step`), where its ring fills with weights while the kernel
        # in front drains (Qwen3-8B sizes, batch 1: 3.60 -> 3.38 ms per step); "1" always, "0" never (with the
        # library's products in between it costs 1 to 2 %: waiting blocks hold SM slots and gain nothing)
        mode = get("ULLM_B200_PDL", "auto")
        self.pdl_mode = {"1": True, "0": False}.get(mode, "auto")
        self.set_pdl(self.pdl_mode is True)
        # blocks the per-request decode attention aims for when it splits the requests' key ranges
        self.decode_split_target = int(get("ULLM_B200_DECODE_SPLIT_TARGET", "400"))
        # prompt attention on the tcgen05 tensor cores (head size 128); 0: the mma.sync kernel
        # prompt attention at head size 128: "1" the tcgen05 kernels (two query tiles per block where a request
        # brings more than one tile, else one), "pair" / "single" one of them always, "0" the mma.sync kernel
        self.tc_attention_mode = get("ULLM_B200_TC_ATTN", "1")
        self.use_tcgen05_attention = self.tc_attention_mode != "0"
        # the splits of a request's keys merge inside a thread-block cluster (at most 8 splits) instead of through
        # scratch arrays and a second kernel
        # ("auto": for steps of at most 8 rows; "1" / "0": always / never, with `decode_split_target` splits)
        mode = get("ULLM_B200_DECODE_CLUSTER", "auto")
        self.decode_cluster_merge = {"1": True, "0": False}.get(mode, "auto")
        # decode steps: the per-request decode attention kernel applies the q/k norm and the rotation and writes the
        # new key and value itself (one launch less per layer)
        self.fuse_decode_rope = get("ULLM_B200_FUSE_DECODE_ROPE", "1") == "1"
        # a mixed step's leading one-token entries go to the decode attention kernel from this many on (0: never)
        self.mixed_decode_rows = int(get("ULLM_B200_MIXED_DECODE_ROWS", "4"))
        # decode attention on the tcgen05 tensor cores (head size 128), the batch's keys cut evenly over the blocks
        self.use_tcgen05_decode = get("ULLM_B200_DECODE_TC", "0") == "1"
        # decode attention: the batch's keys cut evenly over the warps (True), every request split alike (False),
        # or "auto": the first for batches of very unequal lengths (the mixer says so), else the second
        mode = get("ULLM_B200_DECODE_BALANCED", "auto")
        self.use_balanced_decode = {"1": True, "0": False}.get(mode, "auto")
        # few-row products: "auto" (the default) the weight-streaming TMA kernel for small weights, where a step is
        # bound by launches and start-up and not by memory (measured at Qwen3-0.6B sizes: a decode step of 4 to 16
        # requests 6 to 17 % faster), the library otherwise; "0" always the library; "stream" that kernel always
        # (M <= 32), "skinny" the mma.sync streaming kernel (M <= 32), "tcgen05" (or "1") the stream-K tcgen05
        # kernel (M <= 64)
        mode = get("ULLM_B200_SMALL_M_LINEAR", "auto")
        self.small_m_mode = {"1": "tcgen05", "0": None, "": "auto"}.get(mode, mode)
        # "auto": rows up to which EVERY product of a step is the stream kernel (with dependent launch it beats
        # the library there: Qwen3-8B sizes, 8 requests 4.14 -> 3.60 ms per step, 1 request 3.63 -> 3.32, 16 requests
        # 4.68 -> 4.58)
        self.stream_all_rows = int(get("ULLM_B200_STREAM_ALL_ROWS", "16"))
        # in those steps a block folds its feed-forward norm between the output projection and the gate / up
        # product (one kernel less per layer); 0: the norm stays a kernel of its own
        # 0: norms stay kernels of their own; 1: a block's feed-forward norm is folded between its products in
        # small decode steps; 2: the next block's first norm too (behind this block's last product)
        self.chain_norms = int(get("ULLM_B200_CHAIN_NORMS", "2"))
        if self.small_m_mode not in (None, "auto", "tcgen05", "skinny", "stream"):
            raise KernelError(f"ULLM_B200_SMALL_M_LINEAR={mode!r}: auto, 0, stream, skinny or tcgen05")
        self.stream_weight_bytes = int(get("ULLM_B200_STREAM_WEIGHT_MB", "16")) << 20  # "auto": weights up to this
        self.stream_rows = 32  # rows the stream product takes
        # rows from which the gated feed-forward's first product runs on the own tcgen05 kernel with the activation
        # fused (0 rows would mean always; a huge number never)
        self.fused_mlp_rows = int(get("ULLM_B200_FUSED_MLP_ROWS", "4096"))
        # rows up to which the library's product is called through cuBLASLt with a timed choice of algorithm
        self.lt_rows = int(get("ULLM_B200_LT_ROWS", str(1 << 30)))
        # rows up to which a step runs the second half of a layer (output projection, residual, norm, gated
        # feed-forward, residual) as one cooperative kernel; 0 (the default): never.  Measured at Qwen3-8B sizes:
        # 71 us against 70 us for the separate kernels at 8 rows, 77 against 70 at 16: no gain yet.
        self.fused_tail_rows = int(get("ULLM_B200_FUSED_TAIL_ROWS", "0"))

    # -- ctypes signatures --------------------------------------------------
    def _declare(self) -> None:
        L = self.lib
        P, I, F, LL = c_void_p, c_int, c_float, c_longlong
        sig = {
            "ullm_embedding": [I, P, P, P, I, I, I, P, P, P, P, P],
            "ullm_gather_rows": [I, P, P, P, I, I, I, P, P],
            "ullm_add_rmsnorm": [I, P, P, P, P, I, I, F, P],
            "ullm_act_mul": [I, I, P, P, I, I, P],
            "ullm_cast_bf16_f32": [P, P, LL, P],
            "ullm_qk_norm_rope_store": [I, P, I, I, I, I, P, P, F, P, P, I, I, P, P, P, P, LL, P, P],
            "ullm_qk_norm_in_place": [I, P, I, I, I, I, P, P, F, P, P],
            "ullm_paged_attention_generic": [I, P, LL, P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, LL, P, P],
            "ullm_decode_attention": [P, LL, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, LL, P, P],
            "ullm_decode_attention_balanced": [P, LL, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, F, LL, P, P],
            "ullm_decode_attention_fused": [P, LL, P, P, P, I, P, P, P, P, I, I, I, I, I, I, F, I, LL, P, P, F, P, P, I,
                                            P, P, P, P],
            "ullm_prefill_attention": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P],
            "ullm_prefill_attention_tcgen05": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P],
            "ullm_prefill_attention_pair": [P, LL, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, LL, P, P],
            "ullm_linear_tcgen05": [P, P, P, P, I, I, I, I, I, P, LL, P, I, P, P],
            "ullm_linear_skinny": [P, P, P, P, I, I, I, I, I, P],
            "ullm_linear_stream": [P, P, P, P, P, I, I, I, I, I, P, P],
            "ullm_linear_stream_norm": [P, P, P, P, P, I, I, I, I, I, P, P, P, P, I, I, F, P, P],
            "ullm_layer_tail_fused": [P, P, P, P, P, P, P, P, F, I, I, I, I, I, P, P, P, P],
            "ullm_linear_tcgen05_large": [P, P, P, P, I, I, I, I, I, I, P, P],
            "ullm_decode_attention_tcgen05": [P, LL, P, P, P, I, P, P, P, P, P, P, I, I, I, I, I, I, F, LL, P, P],
            "ullm_lt_linear": [P, P, P, I, I, I, I, P, LL, I, P, LL, P],
            "ullm_argmax": [P, LL, I, I, P, P],
            "ullm_sample": [P, LL, I, I, P, P, P, P, P, P, P, P, P, P],
        }
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = c_int
        L.ullm_wait_selftest.argtypes = [I, P, P, P]
        L.ullm_wait_selftest.restype = c_int
        L.ullm_decode_attention_supported.argtypes = [I, I, I]
        L.ullm_decode_attention_supported.restype = c_int
        L.ullm_decode_attention_balanced_supported.argtypes = [I, I, I, I, I]
        L.ullm_decode_attention_balanced_supported.restype = c_int
        L.ullm_decode_attention_balanced_scratch_floats.argtypes = [I, I]
        L.ullm_decode_attention_balanced_scratch_floats.restype = c_longlong
        L.ullm_decode_attention_tcgen05_supported.argtypes = [I, I, I, I, I]
        L.ullm_decode_attention_tcgen05_supported.restype = c_int
        L.ullm_decode_attention_tcgen05_scratch_floats.argtypes = [I]
        L.ullm_decode_attention_tcgen05_scratch_floats.restype = c_longlong
        L.ullm_decode_attention_cluster_merge.argtypes = [I]
        L.ullm_decode_attention_cluster_merge.restype = None
        L.ullm_decode_attention_last_used_cluster.argtypes = []
        L.ullm_decode_attention_last_used_cluster.restype = c_int
        L.ullm_sample_force_one_block.argtypes = [I]
        L.ullm_sample_force_one_block.restype = None
        L.ullm_sample_last_used_cluster.argtypes = []
        L.ullm_sample_last_used_cluster.restype = c_int
        L.ullm_lt_available.argtypes = []
        L.ullm_lt_available.restype = c_int
        L.ullm_lt_last_choice.argtypes = [P, P, P, P]
        L.ullm_lt_last_choice.restype = None
        L.ullm_prefill_attention_supported.argtypes = [I, I, I]
        L.ullm_prefill_attention_supported.restype = c_int
        L.ullm_prefill_attention_tcgen05_supported.argtypes = [I, I, I, I]
        L.ullm_prefill_attention_tcgen05_supported.restype = c_int
        L.ullm_prefill_attention_tcgen05_blocks_per_sm.restype = c_int
        L.ullm_prefill_attention_pair_supported.argtypes = [I, I, I, I]
        L.ullm_prefill_attention_pair_supported.restype = c_int
        L.ullm_set_pdl.argtypes = [I]
        L.ullm_set_pdl.restype = None
        L.ullm_linear_tcgen05_supported.argtypes = [I, I, I]
        L.ullm_linear_tcgen05_supported.restype = c_int
        L.ullm_linear_tcgen05_blocks.restype = c_int
        L.ullm_linear_tcgen05_large_supported.argtypes = [I, I, I]
        L.ullm_linear_tcgen05_large_supported.restype = c_int
        L.ullm_linear_skinny_supported.argtypes = [I, I, I]
        L.ullm_linear_skinny_supported.restype = c_int
        L.ullm_layer_tail_fused_supported.argtypes = [I, I, I, I]
        L.ullm_layer_tail_fused_supported.restype = c_int
        L.ullm_layer_tail_fused_scratch_floats.argtypes = [I]
        L.ullm_layer_tail_fused_scratch_floats.restype = c_longlong
        L.ullm_layer_tail_fused_counters.argtypes = [I]
        L.ullm_layer_tail_fused_counters.restype = c_longlong
        L.ullm_layer_tail_fused_last_grid.restype = c_int
        L.ullm_linear_stream_supported.argtypes = [I, I, I]
        L.ullm_linear_stream_supported.restype = c_int
        L.ullm_linear_stream_sq_floats.argtypes = [I]
        L.ullm_linear_stream_sq_floats.restype = c_longlong
        L.ullm_linear_stream_blocks_per_sm.argtypes = [I]
        L.ullm_linear_stream_blocks_per_sm.restype = None
        L.ullm_linear_stream_smem_kb.argtypes = [I]
        L.ullm_linear_stream_smem_kb.restype = None
        L.ullm_linear_stream_ksplit_max.argtypes = [I]
        L.ullm_linear_stream_ksplit_max.restype = None

    def _check(self, code: int, what: str) -> None:
        self.launches += 1
        if code != 0:
            raise KernelError(f"{what}: {_ERRORS.get(code, f'error {code}')}")

    def set_pdl(self, on: bool) -> None:
        """Programmatic dependent launch for every kernel of the library: a kernel's launch and
        set-up overlap the tail of the kernel before it in the stream."""
        if bool(on) != self.pdl:
            self.lib.ullm_set_pdl(1 if on else 0)
            self.pdl = bool(on)

    # -- status word ----------------------------------------------------------
    def raise_on_status(self) -> None:
        """Reads the device status word (synchronizes) and raises if a kernel
        refused an out-of-range index since the last call."""
        s = self.status.tolist()
        if s[0] != 0:
            self.status.zero_()
            if self._lin_counters is not None:
                self._lin_counters.zero_()  # a product that gave up may have left tiles half counted
            for _part, _prefix, flags in self._decb.values():
                flags.zero_()  # likewise the merge flags of the balanced decode attention
            for _scratch, counters, _normed in self._tail_ws.values():
                counters.zero_()  # and the tickets and grid barriers of the fused layer tail
            msg = STATUS_MESSAGES.get(s[0], "status {code}").format(index=s[1], value=s[2], code=s[0])
            raise KernelError(f"a kernel refused an index: {msg}")

    def wait_selftest(self, limit: int = 4096) -> int:
        """Runs the kernels' give-up path on purpose (see csrc/wait_selftest.cu): a one-block kernel waits
        `limit` polls on a barrier nobody arrives at, records the timeout in the status word, frees its tensor
        memory and returns.  Returns 1 when the wait ran out; the status word is left set for the caller
        (`raise_on_status` reads and clears it)."""
        out = torch.zeros(1, dtype=torch.int32, device="cuda")
        self._check(self.lib.ullm_wait_selftest(int(limit), _ptr(self.status), _ptr(out), _stream()), "wait_selftest")
        return int(out.item())

    # -- library matrix products ---------------------------------------------
    def small_m_linear(self, x, weight, out, bias=None, act: int | None = None) -> bool:
        """The hand-written tcgen05/TMA product for few rows (decode steps): bfloat16 operands, out bfloat16
        or float32; with `act` (0 silu, 1 gelu_tanh) weight stacks gate rows on up rows and out is
        act(gate) * up.  False when the shape is not one it takes (the caller then uses the library)."""
        M, K = x.shape
        N = weight.shape[0]
        n_out = N // 2 if act is not None else N
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32)
                or (bias is not None and bias.dtype != torch.bfloat16) or (act is not None and N % 2)
                or not self.lib.ullm_linear_tcgen05_supported(M, N, K)
                or x.data_ptr() % 16 or weight.data_ptr() % 16):
            return False
        if self._lin_ws is None:
            blocks = self.lib.ullm_linear_tcgen05_blocks()
            if blocks <= 0:
                raise KernelError("linear_tcgen05: cannot read the device's SM count")
            self._lin_ws = torch.empty(blocks * 2 * 64 * 128, dtype=torch.float32, device="cuda")
            self._lin_counters = torch.zeros(16384, dtype=torch.int32, device="cuda")
        code = self.lib.ullm_linear_tcgen05(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), M, N, K,
                                            1 if out.dtype == torch.float32 else 0, 0 if act is None else act + 1,
                                            _ptr(self._lin_ws), self._lin_ws.numel(), _ptr(self._lin_counters),
                                            self._lin_counters.numel(), _ptr(self.status), _stream())
        if code == 4:  # more tiles than counters: the library takes it
            return False
        self._check(code, f"linear_tcgen05 ({M}x{K} . {N}x{K})")
        return True

    def skinny_linear(self, x, weight, out, bias=None, act: int | None = None) -> bool:
        """The streaming mma.sync product for very few rows (M <= 32), same contract as `small_m_linear`."""
        M, K = x.shape
        N = weight.shape[0]
        n_out = N // 2 if act is not None else N
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32)
                or (bias is not None and bias.dtype != torch.bfloat16) or (act is not None and N % 2)
                or not self.lib.ullm_linear_skinny_supported(M, N, K)
                or x.data_ptr() % 16 or weight.data_ptr() % 16):
            return False
        self._check(self.lib.ullm_linear_skinny(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), M, N, K,
                                                1 if out.dtype == torch.float32 else 0,
                                                0 if act is None else act + 1, _stream()),
                    f"linear_skinny ({M}x{K} . {N}x{K})")
        return True

    @_timed("linear", _weight_bytes, skipped=True)
    def stream_linear(self, x, weight, out, bias=None, act: int | None = None, residual=None, norm_behind=None,
                      norm_in_front=None) -> bool:
        """`_stream_linear` as a call of its own (a block that chains its products): booked under the products'
        group."""
        return self._stream_linear(x, weight, out, bias, act, residual, norm_behind, norm_in_front)

    def _stream_linear(self, x, weight, out, bias=None, act: int | None = None, residual=None, norm_behind=None,
                       norm_in_front=None) -> bool:
        """The weight-streaming product for few rows (M <= 32; csrc/linear_stream.cu): a TMA ring per block that
        is filled with weight tiles before the kernel in front has finished (programmatic dependent launch),
        mma.sync on the swizzled tiles.  Same contract as `small_m_linear`; `residual` ([M, n_out], bfloat16;
        may be `out`) is added to the product in 32-bit before the one rounding.

        An RMSNorm between two such products costs no kernel (rmsnorm(r) * w = (1 / rms(r)) * (r * w)):
        `norm_behind=(w, operand, sq)` on the product in front of the norm also writes result * w to `operand`
        ([M, n_out] bfloat16) and the units' sums of squares to `sq` (float32, `stream_sq_floats(n_out)`);
        `norm_in_front=(sq, cols, eps)` on the product behind it (whose x is that operand) multiplies its sums by
        the rows' 1 / rms.  Both for at most 16 rows."""
        M, K = x.shape
        N = weight.shape[0]
        n_out = N // 2 if act is not None else N
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32)
                or (bias is not None and bias.dtype != torch.bfloat16) or (act is not None and N % 2)
                or (residual is not None and (residual.dtype != torch.bfloat16 or residual.shape != (M, n_out)
                                              or not residual.is_contiguous()))
                or not self.lib.ullm_linear_stream_supported(M, N, K)
                or x.data_ptr() % 16 or weight.data_ptr() % 16):
            return False
        pre_w = pre_out = sq_out = sq_in = None
        sq_count, sq_cols, sq_eps = 0, 0, 0.0
        if norm_behind is not None:
            pre_w, pre_out, sq_out = norm_behind
            _need(pre_w, "norm weight", torch.float32)
            _need(pre_out, "normed operand", torch.bfloat16)
            _need(sq_out, "sums of squares", torch.float32)
            if (act is not None or M > 16 or pre_w.numel() != n_out or pre_out.shape != (M, n_out)
                    or sq_out.numel() < self.stream_sq_floats(n_out)):
                raise KernelError("stream_linear: norm_behind needs a plain product of at most 16 rows, a weight per "
                                  "output column, an operand of the output's shape and room for the sums of squares")
        if norm_in_front is not None:
            sq_in, sq_cols, sq_eps = norm_in_front
            _need(sq_in, "sums of squares", torch.float32)
            if M > 16 or sq_cols != K or sq_in.numel() < self.stream_sq_floats(K):
                raise KernelError("stream_linear: norm_in_front needs at most 16 rows and the sums of squares of K columns")
            sq_count = self.stream_sq_floats(K) // 16
        self._check(self.lib.ullm_linear_stream_norm(
            _ptr(x), _ptr(weight), _ptr(bias), _ptr(residual), _ptr(out), M, N, K, 1 if out.dtype == torch.float32 else 0,
            0 if act is None else act + 1, _ptr(pre_w), _ptr(pre_out), _ptr(sq_out), _ptr(sq_in), sq_count, int(sq_cols),
            float(sq_eps), _ptr(self.status), _stream()), f"linear_stream ({M}x{K} . {N}x{K})")
        return True

    def stream_sq_floats(self, n_out: int) -> int:
        """Floats of the sums-of-squares array that `stream_linear(norm_behind=...)` fills for `n_out` columns."""
        return int(self.lib.ullm_linear_stream_sq_floats(int(n_out)))

    def stream_chain_applies(self, rows: int, dtype) -> bool:
        """True for the steps whose products are all the stream kernel (the automatic policy, bfloat16, few rows):
        a block may then chain its products with the norm folded between them."""
        return bool(self.small_m_mode == "auto" and dtype == torch.bfloat16 and rows <= min(self.stream_all_rows, 16)
                    and self.chain_norms > 0)

    def layer_tail_applies(self, rows: int, dtype, hidden: int, attn_width: int, intermediate: int) -> bool:
        """True when `fused_layer_tail` takes these sizes and the switch is on: decode-sized batches (at most
        `fused_tail_rows` rows, never more than 16) in bfloat16."""
        return bool(self.fused_tail_rows > 0 and rows <= min(self.fused_tail_rows, 16) and dtype == torch.bfloat16
                    and self.lib.ullm_layer_tail_fused_supported(rows, hidden, attn_width, intermediate))

    @_timed("layer_tail_fused", lambda self_attn, residual, act_out, w_o, w_gate_up, w_down, *r: (
        w_o.numel() + w_gate_up.numel() + w_down.numel()) * 2)
    def fused_layer_tail(self, attn, residual, act_out, w_o, w_gate_up, w_down, norm_w, eps: float, act: int = 0):
        """The second half of a pre-norm decoder layer in one kernel (csrc/layer_tail_fused.cu):
        residual += attn @ w_o.T;  act_out = act(h @ Wgate.T) * (h @ Wup.T) with h = rmsnorm(residual) * norm_w;
        residual += act_out @ w_down.T.  `residual` [M, H] is updated in place; `act_out` [M, I] is a work buffer.
        bfloat16, M <= 16.  Call `layer_tail_applies` first."""
        M, QD = attn.shape
        H = residual.shape[1]
        inter = act_out.shape[1]
        for t_, n_ in ((attn, "attn"), (residual, "residual"), (act_out, "act_out"), (w_o, "w_o"),
                       (w_gate_up, "w_gate_up"), (w_down, "w_down")):
            _need(t_, n_, torch.bfloat16)
            if t_.data_ptr() % 16:
                raise KernelError(f"fused_layer_tail: {n_} is not 16-byte aligned")
        _need(norm_w, "norm_w", torch.float32)
        if (residual.shape[0] != M or act_out.shape[0] != M or w_o.shape != (H, QD) or w_gate_up.shape != (2 * inter, H)
                or w_down.shape != (H, inter) or norm_w.numel() != H):
            raise KernelError(f"fused_layer_tail: attn {tuple(attn.shape)}, residual {tuple(residual.shape)}, act_out "
                              f"{tuple(act_out.shape)}, w_o {tuple(w_o.shape)}, w_gate_up {tuple(w_gate_up.shape)}, "
                              f"w_down {tuple(w_down.shape)}")
        ws = self._tail_ws.get(H)
        if ws is None:  # scratch of the split units and the zeroed counters, made at the first (eager) call
            ws = (torch.empty(self.lib.ullm_layer_tail_fused_scratch_floats(H), dtype=torch.float32, device="cuda"),
                  torch.zeros(self.lib.ullm_layer_tail_fused_counters(H), dtype=torch.int32, device="cuda"),
                  torch.empty(16, H, dtype=torch.bfloat16, device="cuda"))  # the normed rows between its phases
            self._tail_ws[H] = ws
        self._check(self.lib.ullm_layer_tail_fused(
            _ptr(attn), _ptr(residual), _ptr(act_out), _ptr(ws[2]), _ptr(w_o), _ptr(w_gate_up), _ptr(w_down), _ptr(norm_w),
            float(eps), act + 1, M, H, QD, inter, _ptr(ws[0]), _ptr(ws[1]), _ptr(self.status), _stream()),
            f"layer_tail_fused ({M} rows, hidden {H}, intermediate {inter})")
        return residual

    def large_linear(self, x, weight, out, bias=None, act: int | None = None, variant: int = 0) -> bool:
        """The persistent tcgen05/TMA product for many rows (prompt portions): tiles of 128 x 256, two accumulators
        in tensor memory, bias and the gate activation in the epilogue.  Same contract as `small_m_linear`."""
        M, K = x.shape
        N = weight.shape[0]
        n_out = N // 2 if act is not None else N
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, n_out) or out.dtype not in (torch.bfloat16, torch.float32)
                or (bias is not None and bias.dtype != torch.bfloat16) or (act is not None and N % 2)
                or not self.lib.ullm_linear_tcgen05_large_supported(M, N, K)
                or x.data_ptr() % 16 or weight.data_ptr() % 16 or out.data_ptr() % 16):
            return False
        self._check(self.lib.ullm_linear_tcgen05_large(_ptr(x), _ptr(weight), _ptr(bias), _ptr(out), M, N, K,
                                                       1 if out.dtype == torch.float32 else 0,
                                                       0 if act is None else act + 1, variant, _ptr(self.status),
                                                       _stream()),
                    f"linear_tcgen05_large ({M}x{K} . {N}x{K})")
        return True

    def lt_linear(self, x, weight, out, tune: bool = True) -> bool:
        """out = x @ weight.T through cuBLASLt with a measured choice among the library's candidate algorithms
        (timed once per shape, outside stream captures, with L2 flushed; kept for the life of the process).
        bfloat16 operands, bfloat16 or float32 out, no bias.  False: not taken (the caller uses torch)."""
        M, K = x.shape
        N = weight.shape[0]
        if (x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_contiguous()
                or not weight.is_contiguous() or not out.is_contiguous() or weight.shape[1] != K
                or out.shape != (M, N) or out.dtype not in (torch.bfloat16, torch.float32) or K % 8
                or (out.dtype == torch.bfloat16 and N % 8)
                or x.data_ptr() % 16 or weight.data_ptr() % 16 or out.data_ptr() % 16):
            return False
        if self._lt_ok is None:
            self._lt_ok = bool(self.lib.ullm_lt_available())
            if self._lt_ok:
                self._lt_ws = torch.empty(32 << 20, dtype=torch.uint8, device="cuda")
        if not self._lt_ok:
            return False
        out_f32 = 1 if out.dtype == torch.float32 else 0
        key = (M, N, K, out_f32)
        flush = None
        if tune and key not in self._lt_tuned and not torch.cuda.is_current_stream_capturing():
            try:
                flush = torch.zeros(256 << 20, dtype=torch.uint8, device="cuda")  # larger than L2; gone after this call
            except torch.cuda.OutOfMemoryError:
                flush = None  # no room to time anything: the library's first candidate it is
            self._lt_tuned.add(key)
        rc = self.lib.ullm_lt_linear(_ptr(x), _ptr(weight), _ptr(out), M, N, K, out_f32, _ptr(self._lt_ws),
                                     self._lt_ws.numel(), 1 if flush is not None else 0, _ptr(flush),
                                     0 if flush is None else flush.numel(), _stream())
        if rc == 4:  # a shape the library has no candidate for
            return False
        self._check(rc, f"lt_linear ({M}x{K} . {N}x{K})")
        return True

    def _lt_takes(self, rows: int, weight) -> bool:
        """Products that go through the timed choice: weights of at least 8 MB (below that there is nothing to
        gain and a timing pass per shape to lose) at the padded row counts of decode steps (1, 2, 4, 8, 16, 32, 48,
        64) and at whole multiples of 256 rows (full prompt portions).  Other row counts would each cost a timing pass for a shape that may
        never come again; they take the library's own first choice."""
        if rows > self.lt_rows or weight.numel() < (1 << 22):
            return False
        return rows in (1, 2, 4, 8) or rows % 16 == 0 and (rows <= 64 or rows % 256 == 0)

    def lt_last_choice(self) -> dict:
        """The last timed choice: index in the library's list, candidates, microseconds (chosen, list's first)."""
        c, n = c_int(0), c_int(0)
        b, f = c_float(0), c_float(0)
        self.lib.ullm_lt_last_choice(ctypes.byref(c), ctypes.byref(n), ctypes.byref(b), ctypes.byref(f))
        return {"chosen": c.value, "candidates": n.value, "best_us": b.value, "first_us": f.value}

    def _own_linear(self, x, weight, out, bias=None, act=None) -> bool:
        """Tries the hand-written few-row product that the mode names; False: the caller uses the library."""
        if self.small_m_mode == "skinny":
            return x.shape[0] <= 32 and self.skinny_linear(x, weight, out, bias, act)
        if self.small_m_mode == "stream":
            return x.shape[0] <= self.stream_rows and self._stream_linear(x, weight, out, bias, act)
        if self.small_m_mode == "auto":
            rows = x.shape[0]
            return (rows <= self.stream_rows
                    and (rows <= self.stream_all_rows
                         or weight.numel() * weight.element_size() <= self.stream_weight_bytes)
                    and self._stream_linear(x, weight, out, bias, act))
        if self.small_m_mode == "tcgen05":
            if x.shape[0] <= 64:
                return self.small_m_linear(x, weight, out, bias, act)
            return self.large_linear(x, weight, out, bias, act)
        return False

    @_timed("linear", _weight_bytes)
    def linear(self, x, weight, out, bias=None):
        """out = x @ weight.T (+ bias).  Few bfloat16 rows: a hand-written kernel when one is switched on.
        Otherwise the vendor library's matrix product, float32 without any reduced-precision mode."""
        _need(x, "x")
        _need(out, "out")
        if self._own_linear(x, weight, out, bias):
            return out
        if bias is None and self._lt_takes(x.shape[0], weight) and self.lt_linear(x, weight, out):
            return out
        if bias is not None:
            torch.addmm(bias, x, weight.t(), out=out)
        else:
            torch.mm(x, weight.t(), out=out)
        return out

    @_timed("linear_gate_up_act", _weight_bytes)
    def linear_act_mul(self, x, weight, out, gate_up, act: int = 0):
        """out[T, I] = act(x @ Wg.T) * (x @ Wu.T) for weight = [Wg; Wu] ([2 I, K]).  Few bfloat16 rows: one
        kernel, the activation in the product's epilogue (gate and up never leave the chip).  Otherwise the
        product into `gate_up` [T, 2 I] and the activation kernel."""
        _need(x, "x")
        _need(out, "out")
        if self._own_linear(x, weight, out, None, act):
            return out
        # many rows: the persistent tcgen05 product with the activation in its epilogue against the library's
        # product followed by the activation kernel (measured at Qwen3-8B sizes): 300 against 310 us at 2,048 rows
        # with the library's own first algorithm, but 300 against 251 + 31 us with the library's timed choice
        # (`lt_linear`); 576 against 500 - 535 + 62 us at 4,096 rows, from where it is taken
        if x.shape[0] >= self.fused_mlp_rows and self.large_linear(x, weight, out, None, act):
            return out
        self.linear(x, weight, gate_up)
        self.act_mul(gate_up, out, act)
        return out

    @_timed("linear_head", _weight_bytes)
    def linear_f32_out(self, x, weight, out):
        """out (float32) = x @ weight.T for x/weight in float32 or bfloat16."""
        _need(out, "out", torch.float32)
        if x.dtype == torch.float32:
            torch.mm(x, weight.t(), out=out)
            return out
        if self._own_linear(x, weight, out):
            return out
        if self._lt_takes(x.shape[0], weight) and self.lt_linear(x, weight, out):
            return out
        if self._f32_out_mm is None:
            try:
                torch.mm(x[:1], weight[:8].t(), out_dtype=torch.float32)
                self._f32_out_mm = True
            except (TypeError, RuntimeError):
                self._f32_out_mm = False
        if self._f32_out_mm:
            torch.mm(x, weight.t(), out_dtype=torch.float32, out=out)
        else:
            tmp = torch.mm(x, weight.t())
            self._check(self.lib.ullm_cast_bf16_f32(_ptr(tmp), _ptr(out), tmp.numel(), _stream()), "cast")
        return out

    # -- hand-written kernels ----------------------------------------------------
    @_timed("embedding")
    def embedding(self, ids, table, out, last_tokens=None, token_req=None, req_slots=None):
        """out[t] = table[ids[t]].  With `last_tokens` (and the batch row of each token and the request
        slot of each batch row), an id of -1 means the token that request sampled last."""
        _need(ids, "ids", torch.int32)
        _need(table, "table")
        _need(out, "out", table.dtype)
        T, H = out.shape
        if ids.numel() < T or table.shape[1] != H:
            raise KernelError(f"embedding: ids {tuple(ids.shape)}, table {tuple(table.shape)}, out {tuple(out.shape)}")
        if last_tokens is not None:
            for t_, n_ in ((last_tokens, "last_tokens"), (token_req, "token_req"), (req_slots, "req_slots")):
                _need(t_, n_, torch.int32)
        self._check(self.lib.ullm_embedding(_DT[table.dtype], _ptr(ids), _ptr(table), _ptr(out), T, H,
                                            table.shape[0], _ptr(last_tokens), _ptr(token_req), _ptr(req_slots),
                                            _ptr(self.status), _stream()), "embedding")

    @_timed("gather_rows")
    def gather_rows(self, src, rows, out):
        _need(src, "src")
        _need(rows, "rows", torch.int32)
        _need(out, "out", src.dtype)
        R, C = out.shape
        if src.shape[1] != C or rows.numel() < R:
            raise KernelError(f"gather_rows: src {tuple(src.shape)}, rows {tuple(rows.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_gather_rows(_DT[src.dtype], _ptr(rows), _ptr(src), _ptr(out), R, C, src.shape[0],
                                              _ptr(self.status), _stream()), "gather_rows")

    @_timed("add_rmsnorm")
    def add_rmsnorm(self, x, residual, weight, eps, out):
        _need(x, "x")
        _need(weight, "weight", torch.float32)
        _need(out, "out", x.dtype)
        if residual is not None:
            _need(residual, "residual", x.dtype)
            if residual.shape != x.shape:
                raise KernelError("add_rmsnorm: residual shape differs from x")
        rows, cols = x.shape
        if weight.numel() != cols or out.shape != x.shape:
            raise KernelError(f"add_rmsnorm: x {tuple(x.shape)}, weight {tuple(weight.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_add_rmsnorm(_DT[x.dtype], _ptr(x), _ptr(residual), _ptr(weight), _ptr(out), rows,
                                              cols, float(eps), _stream()), f"add_rmsnorm (row length {cols})")

    @_timed("act_mul")
    def act_mul(self, gate_up, out, act: int = 0):
        _need(gate_up, "gate_up")
        _need(out, "out", gate_up.dtype)
        rows, inter = out.shape
        if gate_up.shape != (rows, 2 * inter):
            raise KernelError(f"act_mul: gate_up {tuple(gate_up.shape)}, out {tuple(out.shape)}")
        self._check(self.lib.ullm_act_mul(_DT[gate_up.dtype], act, _ptr(gate_up), _ptr(out), rows, inter, _stream()),
                    "act_mul")

    def check_attention_sizes(self, *a):
        check_attention_sizes(*a)

    @_timed("qk_norm_rope_store")
    def qk_norm_rope_store(self, qkv, num_q, num_kv, head_dim, q_w, k_w, eps, cos, sin, rotary_dim, positions,
                           slot_mapping, k_pages, v_pages):
        _need(qkv, "qkv")
        T, W = qkv.shape
        if W != (num_q + 2 * num_kv) * head_dim:
            raise KernelError(f"qk_norm_rope_store: qkv row length {W} != (Hq + 2 Hkv) * D")
        for t, n in ((q_w, "q_norm weight"), (k_w, "k_norm weight"), (cos, "cos table"), (sin, "sin table")):
            if t is not None:
                _need(t, n, torch.float32)
        max_pos = 0
        if rotary_dim > 0:
            if cos is None or sin is None or cos.shape != sin.shape or cos.shape[1] != rotary_dim // 2:
                raise KernelError("qk_norm_rope_store: cos/sin tables must be [positions, rotary_dim / 2]")
            max_pos = cos.shape[0]
            _need(positions, "positions", torch.int32)
        num_slots = 0
        if slot_mapping is not None:
            _need(slot_mapping, "slot_mapping", torch.int32)
            _need(k_pages, "k_pages", qkv.dtype)
            _need(v_pages, "v_pages", qkv.dtype)
            if k_pages.shape[-2:] != (num_kv, head_dim) or v_pages.shape != k_pages.shape:
                raise KernelError(f"qk_norm_rope_store: pages {tuple(k_pages.shape)} do not end in (Hkv, D)")
            num_slots = k_pages.numel() // (num_kv * head_dim)
        self._check(self.lib.ullm_qk_norm_rope_store(
            _DT[qkv.dtype], _ptr(qkv), T, num_q, num_kv, head_dim, _ptr(q_w), _ptr(k_w), float(eps), _ptr(cos),
            _ptr(sin), rotary_dim, max_pos, _ptr(positions), _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages),
            num_slots, _ptr(self.status), _stream()), f"qk_norm_rope_store (head_dim {head_dim})")

    @_timed("qk_norm_rope_store")
    def qk_norm_in_place(self, qkv, num_q, num_kv, head_dim, q_w, k_w, eps):
        """Per-head RMSNorm of the queries and the keys of `qkv` ([T, (Hq + 2 Hkv) D]) where they lie; nothing is
        stored in a cache.  (For a position encoding with code of its own, which then changes q and k.)"""
        _need(qkv, "qkv")
        T, W = qkv.shape
        if W != (num_q + 2 * num_kv) * head_dim:
            raise KernelError(f"qk_norm_in_place: qkv row length {W} != (Hq + 2 Hkv) * D")
        for t, n in ((q_w, "q_norm weight"), (k_w, "k_norm weight")):
            if t is not None:
                _need(t, n, torch.float32)
        self._check(self.lib.ullm_qk_norm_in_place(_DT[qkv.dtype], _ptr(qkv), T, num_q, num_kv, head_dim, _ptr(q_w),
                                                   _ptr(k_w), float(eps), _ptr(self.status), _stream()),
                    f"qk_norm_in_place (head_dim {head_dim})")

    def _decode_choice(self, T, ragged, num_q, num_kv, head_dim, page_size, row_stride) -> str:
        """Which decode attention kernel takes T one-token rows: "tcgen05", "balanced" or "split"."""
        balanced = ragged if self.use_balanced_decode == "auto" else self.use_balanced_decode
        if (self.use_tcgen05_decode and self.lib.ullm_decode_attention_tcgen05_supported(
                head_dim, num_q, num_kv, T, page_size) and row_stride % head_dim == 0):
            return "tcgen05"
        if balanced and self.lib.ullm_decode_attention_balanced_supported(head_dim, num_q, num_kv, T, page_size):
            return "balanced"
        return "split"

    def decode_fusion_applies(self, ctx, qkv, num_q, num_kv, head_dim, page_size, rotary_dim, cos,
                              ragged: bool = False) -> bool:
        """True when the step's attention is the per-request decode kernel and that kernel can prepare q, k and v
        itself (norm, rotation, cache write): the caller then skips `qk_norm_rope_store` and hands the pieces to
        `paged_attention(..., fuse=...)`."""
        T = qkv.shape[0]
        return bool(self.fuse_decode_rope and ctx is not None and ctx.decode_only and T == ctx.num_requests
                    and qkv.dtype == torch.bfloat16 and cos is not None and rotary_dim == head_dim
                    and self.lib.ullm_decode_attention_supported(head_dim, num_q, num_kv)
                    and self._decode_choice(T, ragged, num_q, num_kv, head_dim, page_size,
                                            qkv.stride(0)) == "split")

    def _decode_rows(self, qkv, out, k_pages, v_pages, block_table, req_slots, kv_len, num_q, num_kv, head_dim,
                     page_size, window, scale, num_pages, ragged, ctx, fuse=None) -> None:
        """Decode attention of T one-token rows (row i belongs to request row i): streams the pages once."""
        T = out.shape[0]
        choice = self._decode_choice(T, ragged, num_q, num_kv, head_dim, page_size, qkv.stride(0))
        if fuse is not None and choice != "split":
            raise KernelError("decode attention: q and k were left unprepared for a kernel that does not prepare them")
        tc = choice == "tcgen05"
        if choice != "split":
            # both kernels cut the batch's keys evenly (over blocks, over warps) and share the scratch arrays
            # and the merge kernel for the pairs that a cut went through
            key = (head_dim, num_q, num_kv)
            if key not in self._decb:
                n = self.lib.ullm_decode_attention_balanced_scratch_floats(head_dim, num_q // num_kv)
                if head_dim == 128:
                    n = max(n, self.lib.ullm_decode_attention_tcgen05_scratch_floats(num_q // num_kv))
                if n <= 0:
                    raise KernelError("decode attention: cannot size its grid on this device")
                self._decb[key] = (torch.empty(n, dtype=torch.float32, device="cuda"),
                                   torch.zeros(513, dtype=torch.int32, device="cuda"),
                                   torch.zeros(512 * num_q, dtype=torch.int32, device="cuda"))
            part, prefix, flags = self._decb[key]
            fn = self.lib.ullm_decode_attention_tcgen05 if tc else self.lib.ullm_decode_attention_balanced
            self._check(fn(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(out), _ptr(part), _ptr(prefix), _ptr(flags), T, num_q, num_kv, head_dim,
                page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream()),
                f"decode_attention_{'tcgen05' if tc else 'balanced'} (head_dim {head_dim})")
            self.launches += 1  # the merge of the shared pairs
            self.attention_path = "decode_tcgen05" if tc else "decode_balanced"
            return
        # Up to 8 rows (the steps that run under dependent launch) the splits of a request merge inside a
        # thread-block cluster: no merge kernel stands between the attention and the output projection, whose ring
        # fills meanwhile.  The cluster is the largest power of two that keeps all blocks in one wave of two per
        # SM (8 requests x 8 kv heads: 4 splits, 3.59 ms per step against 3.87 with 7 splits and the merge kernel;
        # 3, 5, 6, 7 and 8 splits: 3.70, 4.06, 3.98, 3.93, 4.06).  More rows: splits by `decode_split_target`,
        # merged by the second kernel.
        cluster = T <= max(8, self.stream_all_rows) if self.decode_cluster_merge == "auto" else self.decode_cluster_merge
        self.lib.ullm_decode_attention_cluster_merge(1 if cluster else 0)
        if cluster and self.decode_cluster_merge == "auto":
            splits = 8
            while splits > 1 and T * num_kv * splits > 2 * self.sm_count:
                splits //= 2
        else:
            splits = max(1, min(8 if cluster else 32, -(-self.decode_split_target // (T * num_kv))))
            # (request, kv head) pairs that fill half of the places on the SMs or more (two blocks per SM), but not
            # more than all of them, run unsplit: one wave, no merge launch (24 x 2,048 tokens, 8 kv heads: 46 us
            # against 50 with 3 splits and 58 with 2; 32 x 2,048: 52 against 61 with 2 splits)
            if self.decode_cluster_merge == "auto" and self.sm_count <= T * num_kv <= 2 * self.sm_count:
                splits = 1
        # (splits x rows stays below the blocks aimed for, per kv head, plus one split per row)
        most = num_q * (self.decode_split_target // num_kv + max(T, getattr(ctx.workspace, "max_requests", 0)))
        scratch = ctx.workspace.get("attn.decode_scratch", T * num_q * splits, head_dim + 2, torch.float32,
                                    reserve=most)
        if fuse is not None:
            for t, n in ((fuse["cos"], "cos table"), (fuse["sin"], "sin table")):
                _need(t, n, torch.float32)
            _need(fuse["positions"], "positions", torch.int32)
            self._check(self.lib.ullm_decode_attention_fused(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(out), _ptr(scratch), T, num_q, num_kv, head_dim, page_size,
                int(window), float(scale), splits, num_pages, _ptr(fuse["q_w"]), _ptr(fuse["k_w"]), float(fuse["eps"]),
                _ptr(fuse["cos"]), _ptr(fuse["sin"]), fuse["cos"].shape[0], _ptr(fuse["positions"]),
                _ptr(fuse["slot_mapping"]), _ptr(self.status), _stream()),
                f"decode_attention_fused (head_dim {head_dim})")
        else:
            self._check(self.lib.ullm_decode_attention(
                _ptr(qkv), qkv.stride(0), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), block_table.shape[1],
                _ptr(req_slots), _ptr(kv_len), _ptr(out), _ptr(scratch), T, num_q, num_kv, head_dim, page_size,
                int(window), float(scale), splits, num_pages, _ptr(self.status), _stream()),
                f"decode_attention (head_dim {head_dim})")
        if splits > 1 and not self.lib.ullm_decode_attention_last_used_cluster():
            self.launches += 1  # the merge of the splits
        self.attention_path = "decode"
        return

    @_timed("attention")
    def paged_attention(self, qkv, out, k_pages, v_pages, block_table, req_slots, cu_q, kv_len, token_req, num_q, num_kv,
                        head_dim, page_size, window, scale, ctx=None, fuse=None, ragged: bool = False):
        """Attention of every row of the flat batch over its request's pages.
        `qkv` holds q in its first num_q * head_dim columns.  `fuse` (only after `decode_fusion_applies` said
        yes): q, k and v are as the projection left them, and the kernel norms, rotates and stores them itself;
        a dict with q_w, k_w (or None), eps, cos, sin, positions, slot_mapping (or None).  `ragged` (decode
        steps): the caller found the requests' lengths very unequal, which picks the batch-balanced kernel."""
        _need(qkv, "qkv")
        _need(out, "out", qkv.dtype)
        _need(k_pages, "k_pages", qkv.dtype)
        _need(v_pages, "v_pages", qkv.dtype)
        for t, n in ((block_table, "block_table"), (req_slots, "req_slots"), (cu_q, "cu_q"), (kv_len, "kv_len"), (token_req, "token_req")):
            _need(t, n, torch.int32)
        T = out.shape[0]
        if out.shape[1] != num_q * head_dim or qkv.shape[0] < T:
            raise KernelError(f"paged_attention: out {tuple(out.shape)}, qkv {tuple(qkv.shape)}")
        if k_pages.shape[-3:] != (page_size, num_kv, head_dim):
            raise KernelError(f"paged_attention: pages {tuple(k_pages.shape)} != [*, {page_size}, {num_kv}, {head_dim}]")
        num_pages = k_pages.numel() // (page_size * num_kv * head_dim)
        decode_ok = (ctx is not None and qkv.dtype == torch.bfloat16
                     and self.lib.ullm_decode_attention_supported(head_dim, num_q, num_kv))
        if decode_ok and ctx.decode_only and T == ctx.num_requests:
            self._decode_rows(qkv, out, k_pages, v_pages, block_table, req_slots, kv_len, num_q, num_kv, head_dim,
                              page_size, window, scale, num_pages, ragged, ctx, fuse)
            return
        if fuse is not None:
            raise KernelError("paged_attention: q and k were left unprepared, but this step is no decode step")
        # A step that mixes decoded tokens with prompt portions: the one-token entries at its head (the scheduler
        # puts them first) go to the decode kernel, which streams their pages once; the prompt kernels would give
        # each of them a 128-row tile of its own.  The rest of the step follows with its own slices of the
        # per-request arrays (cu_q holds absolute rows, so q and out stay whole).
        n_dec = 0
        if decode_ok and self.mixed_decode_rows > 0 and getattr(ctx, "cu_q_host", None) is not None:
            cq = ctx.cu_q_host
            while n_dec < ctx.num_requests and cq[n_dec] == n_dec and cq[n_dec + 1] == n_dec + 1:
                n_dec += 1
            if n_dec < self.mixed_decode_rows or n_dec == ctx.num_requests:
                n_dec = 0
        if n_dec:
            lens = [ctx.start_positions_host[i] + 1 for i in range(n_dec)]
            ragged = n_dec > 1 and 2 * n_dec * max(lens) > 3 * sum(lens)
            self._decode_rows(qkv[:n_dec], out[:n_dec], k_pages, v_pages, block_table, req_slots[:n_dec], kv_len[:n_dec],
                              num_q, num_kv, head_dim, page_size, window, scale, num_pages, ragged, ctx)
            req_slots, cu_q, kv_len = req_slots[n_dec:], cu_q[n_dec:], kv_len[n_dec:]
        num_requests = (ctx.num_requests - n_dec) if ctx is not None else 0
        pair = single = False
        if ctx is not None and qkv.dtype == torch.bfloat16 and self.use_tcgen05_attention and qkv.stride(0) % head_dim == 0:
            pair = bool(self.tc_attention_mode != "single"
                        and self.lib.ullm_prefill_attention_pair_supported(head_dim, num_q, num_kv, page_size))
            single = bool(not pair and self.lib.ullm_prefill_attention_tcgen05_supported(head_dim, num_q, num_kv, page_size))
        if pair or single:
            entry = self.lib.ullm_prefill_attention_pair if pair else self.lib.ullm_prefill_attention_tcgen05
            self.prefill_attention_kernel = "pair" if pair else "single"
            self._check(entry(
                _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), T, num_requests, num_q, num_kv,
                head_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream()),
                f"prefill_attention_tcgen05 (head_dim {head_dim})")
            self.attention_path = "prefill_tcgen05"
            self.tcgen05_attention_blocks_per_sm = self.lib.ullm_prefill_attention_tcgen05_blocks_per_sm()
            return
        if (ctx is not None and qkv.dtype == torch.bfloat16
                and self.lib.ullm_prefill_attention_supported(head_dim, num_q, num_kv)):
            self._check(self.lib.ullm_prefill_attention(
                _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
                block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), T, num_requests, num_q, num_kv,
                head_dim, page_size, int(window), float(scale), num_pages, _ptr(self.status), _stream()),
                f"prefill_attention (head_dim {head_dim})")
            self.attention_path = "prefill"
            return
        if n_dec:
            raise KernelError("paged_attention: a step's decode rows were split off but no prompt kernel takes the rest")
        self.attention_path = "generic"
        self._check(self.lib.ullm_paged_attention_generic(
            _DT[qkv.dtype], _ptr(qkv), qkv.stride(0), _ptr(out), _ptr(k_pages), _ptr(v_pages), _ptr(block_table),
            block_table.shape[1], _ptr(req_slots), _ptr(cu_q), _ptr(kv_len), _ptr(token_req), T, num_q, num_kv, head_dim, page_size,
            int(window), float(scale), num_pages, _ptr(self.status), _stream()),
            f"paged_attention (head_dim {head_dim})")

    @_timed("sampling")
    def argmax(self, logits, out):
        _need(logits, "logits", torch.float32, contiguous=False)
        _need(out, "out", torch.int32)
        R, V = logits.shape
        if logits.stride(1) != 1 or out.numel() < R:
            raise KernelError("argmax: logits rows must be contiguous and out must hold one id per row")
        self._check(self.lib.ullm_argmax(_ptr(logits), logits.stride(0), R, V, _ptr(out), _stream()), "argmax")

    def set_decode_cluster_merge(self, on: bool) -> None:
        """The splits of the per-request decode attention merge inside a cluster (True) or through scratch arrays
        and the merge kernel (False; tests compare the two), or "auto": the first for one or two requests."""
        self.decode_cluster_merge = on if on == "auto" else bool(on)

    def sample_force_one_block(self, on: bool) -> None:
        """Rows go to the one-block sampling kernel instead of the cluster kernel (tests compare the two)."""
        self.lib.ullm_sample_force_one_block(1 if on else 0)

    def sample_used_cluster(self) -> bool:
        return bool(self.lib.ullm_sample_last_used_cluster())

    @_timed("sampling")
    def sample(self, logits, temperature, top_k, top_p, min_p, uniform, out, probs_out=None, row_slots=None,
               last_tokens=None):
        _need(logits, "logits", torch.float32, contiguous=False)
        R, V = logits.shape
        if logits.stride(1) != 1:
            raise KernelError("sample: logits rows must be contiguous")
        for t, n, dt in ((temperature, "temperature", torch.float32), (top_k, "top_k", torch.int32),
                         (top_p, "top_p", torch.float32), (min_p, "min_p", torch.float32),
                         (uniform, "uniform", torch.float32), (out, "out", torch.int32)):
            _need(t, n, dt)
            if t.numel() < R:
                raise KernelError(f"sample: {n} holds {t.numel()} values for {R} rows")
        if probs_out is not None:
            _need(probs_out, "probs_out", torch.float32)
            if probs_out.shape != (R, V):
                raise KernelError("sample: probs_out must be [rows, vocab]")
        self._check(self.lib.ullm_sample(_ptr(logits), logits.stride(0), R, V, _ptr(temperature), _ptr(top_k),
                                         _ptr(top_p), _ptr(min_p), _ptr(uniform), _ptr(out), _ptr(probs_out),
                                         _ptr(row_slots), _ptr(last_tokens), _stream()), "sample")
