"""Step programs: a model's launches written once, run by one native call per step.

Driving the kernels from Python costs 8 to 10 microseconds of interpreter time per launch (argument checks,
the foreign-function call, an allocation for every intermediate); a prompt step of a 24-layer model has about
200 launches, so each one took at least 3 ms however few tokens it brought. The reference has the same shape
(src/infer/model/qwen2.py:13-52 run from src/infer/engine/model_runner.py:80-97) and the same cost.

A program is built from the model's parts: each part that has an ``emit`` method appends its launches to a
``ProgramBuilder`` instead of running them. A value in a launch record is

* fixed for the model's lifetime: a weight or table (a tensor), a size or constant from the configuration, a
  workspace buffer (``builder.buffer``: activations live in one allocation sized for a number of tokens); or
* a per-step parameter (``builder.param(name, fn)``): ``fn(step)`` is evaluated once per step and its value
  goes into a small table that the records index. The number of tokens, pointers into the step's input
  buffer, the work-unit count of the attention kernel and "does this step take the decode kernel" are such.

``StepProgram.run(step)`` fills the table and calls ``tm_program_run`` (csrc/step_program.cu), which walks the
records and launches. A model with a part that has no ``emit`` (a toy mixer in a test, a part added later)
simply has no program and runs through the parts' ``forward`` methods as before; the two paths launch the
same kernels with the same arguments.
"""

from __future__ import annotations

import ctypes
import struct
from dataclasses import dataclass
from typing import TYPE_CHECKING, Callable

import torch

from . import lib, ops

if TYPE_CHECKING:
    from ..parts.base import StepInputs

OP_ADD_RMSNORM, OP_GEMM_BF16, OP_QKV_ROPE_WRITE = 1, 2, 3
OP_PREFILL_ATTENTION_TC, OP_PREFILL_ATTENTION, OP_DECODE_ATTENTION, OP_SWIGLU = 4, 5, 6, 7
OP_TC_QKV_ROPE_WRITE, OP_TC_LINEAR, OP_DECODE_ATTENTION_UNITS = 8, 9, 10
MAX_ARGS = 24
MIN_TOKENS = 1            # (a caller may keep small steps on the launch-by-launch path by asking for more)
CUBLAS_WORKSPACE = 32 << 20

lib.register_signature("tm_program_op_size", [])
lib.register_signature("tm_program_setup", [ctypes.c_void_p, ctypes.c_longlong])
lib.register_signature("tm_program_run", [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                                          ctypes.c_void_p])


lib.register_signature("tm_program_kind_launches", [ctypes.c_void_p])
KIND_NAMES = {OP_ADD_RMSNORM: "add_rmsnorm", OP_GEMM_BF16: "gemm_bf16", OP_QKV_ROPE_WRITE: "qkv_rope_write",
              OP_PREFILL_ATTENTION_TC: "prefill_attention_tc", OP_PREFILL_ATTENTION: "prefill_attention",
              OP_DECODE_ATTENTION: "decode_attention", OP_SWIGLU: "swiglu", OP_TC_QKV_ROPE_WRITE: "tc_qkv_rope_write",
              OP_TC_LINEAR: "tc_linear", OP_DECODE_ATTENTION_UNITS: "decode_attention_units"}


def kind_launches() -> dict[str, int]:
    """Launches that step programs have issued in this process, by kind of launch."""
    out = (ctypes.c_longlong * 16)()
    lib.load().tm_program_kind_launches(ctypes.addressof(out))
    return {name: int(out[k]) for k, name in KIND_NAMES.items()}


class _Op(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int32), ("cond", ctypes.c_int32), ("param_mask", ctypes.c_uint32),
                ("n_args", ctypes.c_int32), ("arg", ctypes.c_int64 * MAX_ARGS)]


@dataclass(frozen=True)
class Param:
    """A per-step value, by its place in the parameter table."""
    index: int


@dataclass(frozen=True)
class Buffer:
    """Rows of ``row_bytes`` in the program's workspace (as many rows as the program has tokens)."""
    tag: str
    row_bytes: int


@dataclass(frozen=True)
class Float:
    value: float


class ProgramBuilder:
    def __init__(self, device: torch.device, dtype: torch.dtype):
        self.device, self.dtype = device, dtype
        self.ops: list[tuple[int, Param | None, list]] = []
        self._params: dict[str, int] = {}
        self.providers: list[Callable[["StepInputs"], int]] = []
        self.buffers: dict[str, Buffer] = {}
        self.guards: list[Callable[["StepInputs"], bool]] = []
        self.keep: list[torch.Tensor] = []
        self.uses_tc_attention = False

    def param(self, name: str, fn: Callable[["StepInputs"], int]) -> Param:
        """The step parameter of this name (one per name, whoever asks first defines it)."""
        if name not in self._params:
            self._params[name] = len(self.providers)
            self.providers.append(fn)
        return Param(self._params[name])

    def buffer(self, tag: str, row_bytes: int) -> Buffer:
        """A workspace buffer with one row per token. The same tag gives the same buffer: a part names what
        it writes ("normed", "qkv"), and layers, which run one after another, share it."""
        have = self.buffers.get(tag)
        if have is None or have.row_bytes < row_bytes:
            self.buffers[tag] = Buffer(tag, row_bytes)
        return Buffer(tag, row_bytes)

    def guard(self, fn: Callable[["StepInputs"], bool]) -> None:
        """A condition on the step without which the program must not be used for it."""
        self.guards.append(fn)

    def emit(self, kind: int, args: list, cond: Param | None = None) -> None:
        if len(args) > MAX_ARGS:
            raise ValueError(f"a launch record holds {MAX_ARGS} values, not {len(args)}")
        self.ops.append((kind, cond, list(args)))

    # common step parameters
    def tokens(self) -> Param:
        return self.param("n_tokens", lambda s: s.n_tokens)

    def finish(self, capacity: int) -> "StepProgram":
        return StepProgram(self, capacity)


def _float_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", x))[0]


class StepProgram:
    """The launches of one model for steps of up to ``capacity`` tokens."""

    _cublas_workspace: torch.Tensor | None = None

    def __init__(self, b: ProgramBuilder, capacity: int):
        if lib.load().tm_program_op_size() != ctypes.sizeof(_Op):
            raise lib.KernelError("the launch record's layout differs between the library and its binding")
        self.capacity = capacity
        self.device = b.device
        self.providers = b.providers
        self.guards = b.guards
        self.keep = b.keep
        self.uses_tc_attention = b.uses_tc_attention
        offsets, total = {}, 0
        for tag, buf in b.buffers.items():
            offsets[tag] = total
            total += -(-buf.row_bytes * capacity // 256) * 256
        self.workspace = torch.empty(max(total, 256), dtype=torch.uint8, device=b.device)
        base = self.workspace.data_ptr()
        self.ops = (_Op * len(b.ops))()
        for rec, (kind, cond, args) in zip(self.ops, b.ops):
            rec.kind, rec.cond, rec.n_args, mask = kind, (cond.index if cond is not None else -1), len(args), 0
            for i, a in enumerate(args):
                if isinstance(a, Param):
                    mask |= 1 << i
                    rec.arg[i] = a.index
                elif isinstance(a, Buffer):
                    rec.arg[i] = base + offsets[a.tag]
                elif isinstance(a, torch.Tensor):
                    if not a.is_contiguous() or a.device != b.device:
                        raise lib.KernelError("a program takes contiguous tensors on its own device")
                    self.keep.append(a)
                    rec.arg[i] = a.data_ptr()
                elif isinstance(a, Float):
                    rec.arg[i] = _float_bits(a.value)
                elif a is None:
                    rec.arg[i] = 0
                else:
                    rec.arg[i] = int(a)
            rec.param_mask = mask
        self.params = (ctypes.c_int64 * max(1, len(self.providers)))()
        self._report = (ctypes.c_int * 2)(-1, 0)      # failing launch, launches issued
        if StepProgram._cublas_workspace is None:
            StepProgram._cublas_workspace = torch.empty(CUBLAS_WORKSPACE, dtype=torch.uint8, device=b.device)
        ws = StepProgram._cublas_workspace
        lib.call("tm_program_setup", ws.data_ptr(), ws.numel())

    def takes(self, step: "StepInputs", min_tokens: int = MIN_TOKENS) -> bool:
        return min_tokens <= step.n_tokens <= self.capacity and all(g(step) for g in self.guards)

    def run(self, step: "StepInputs") -> None:
        """Launch the step. What the providers read from ``step`` must stay alive until the launches have
        run (the step's tensors do: the caller holds them)."""
        p = self.params
        for i, fn in enumerate(self.providers):
            p[i] = fn(step)
        n = len(self.ops)
        try:
            lib.call("tm_program_run", ctypes.addressof(self.ops), n, ctypes.addressof(p), len(self.providers),
                     ctypes.addressof(self._report), ops._stream())
        except lib.KernelError as e:
            at = self._report[0]
            raise lib.KernelError(f"{e} (launch {at} of {n}, kind {self.ops[at].kind})") from None
        lib.launch_count += self._report[1] - 1          # the call above counted itself once
