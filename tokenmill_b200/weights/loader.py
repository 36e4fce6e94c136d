"""Read a model folder: config.json picks the architecture, safetensors give the tensors by name.

What the reference's loader does (src/infer/model/loader.py:49-131) and this one keeps: every
``*.safetensors`` file of the folder in sorted order; tensors found by name; names the architecture
lists as ignorable are skipped; a missing tensor is an error. What differs: ALL problems are
collected and raised together in one ``WeightError`` that lists missing tensors, unexpected tensors
and wrong shapes; matrices are held in the run's dtype (bfloat16, or float32 on the 32-bit path),
small vectors the kernels read in 32-bit (norm weights, biases) are held in float32, integer tables
in int32.
"""

from __future__ import annotations

import glob
import re
from pathlib import Path

import torch

from ..config.model_config import read_config_json
from ..parts.model import DecoderModel
from ..parts.spec import ModelSpec, WeightSpec
from ..registry import get_architecture


class WeightError(RuntimeError):
    """The checkpoint does not fit the model. ``missing``, ``unexpected`` and ``wrong_shape`` hold
    the full lists; the message shows the first few of each."""

    def __init__(self, folder, missing: list[str], unexpected: list[str], wrong_shape: list[tuple]):
        self.missing, self.unexpected, self.wrong_shape = missing, unexpected, wrong_shape
        parts = [f"checkpoint in {folder} does not fit the model:"]
        if missing:
            parts.append(f"  missing tensors ({len(missing)}): {_head(missing)}")
        if unexpected:
            parts.append(f"  unexpected tensors ({len(unexpected)}): {_head(unexpected)}")
        if wrong_shape:
            shown = [f"{n}: checkpoint {list(got)}, model {list(want)}" for n, got, want in wrong_shape[:8]]
            parts.append(f"  wrong shapes ({len(wrong_shape)}): " + "; ".join(shown)
                         + (" ..." if len(wrong_shape) > 8 else ""))
        super().__init__("\n".join(parts))


def _head(names: list[str], n: int = 8) -> str:
    return ", ".join(names[:n]) + (" ..." if len(names) > n else "")


def resolve_dtype(name: str) -> torch.dtype:
    """auto = bfloat16 (the serving dtype); the reference's auto is float16 on CUDA
    (src/infer/model/loader.py:32-35), which this engine does not run."""
    try:
        return {"auto": torch.bfloat16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
                "float32": torch.float32, "fp32": torch.float32}[name]
    except KeyError:
        raise ValueError(f"dtype must be auto, bfloat16 or float32, got {name!r}") from None


def _target_dtype(spec: WeightSpec, run_dtype: torch.dtype) -> torch.dtype:
    if spec.dtype == "compute":
        return run_dtype
    if spec.dtype == "float32":
        return torch.float32
    if spec.dtype == "int32":
        return torch.int32
    raise ValueError(f"{spec.name}: unknown weight dtype rule {spec.dtype!r}")


def read_spec(folder: str | Path) -> tuple[ModelSpec, object]:
    """(ModelSpec, typed config) of a model folder, through the architecture registry."""
    raw, gen = read_config_json(folder)
    names = raw.get("architectures") or []
    if not names:
        raise ValueError(f"config.json in {folder} names no architecture (key 'architectures')")
    arch = get_architecture(names[0])
    cfg = arch.config_from_dict(raw, gen)
    return arch.build_spec(cfg), cfg


def load_tensors(folder: str | Path, specs: list[WeightSpec], run_dtype: torch.dtype, device: torch.device,
                 ignored_patterns: tuple[str, ...] = ()) -> dict[str, torch.Tensor]:
    from safetensors import safe_open

    folder = Path(folder)
    files = sorted(glob.glob(str(folder / "*.safetensors")))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {folder}")
    want = {s.name: s for s in specs}
    ignore = [re.compile(re.escape(p)) for p in ignored_patterns]
    tensors: dict[str, torch.Tensor] = {}
    unexpected: list[str] = []
    wrong: list[tuple] = []
    for file in files:
        with safe_open(file, framework="pt", device="cpu") as f:
            for name in f.keys():
                spec = want.get(name)
                if spec is None:
                    if not any(p.search(name) for p in ignore):
                        unexpected.append(name)
                    continue
                shape = tuple(f.get_slice(name).get_shape())
                if shape != tuple(spec.shape):
                    wrong.append((name, shape, spec.shape))
                    continue
                t = f.get_tensor(name)
                tensors[name] = t.to(device=device, dtype=_target_dtype(spec, run_dtype)).contiguous()
    missing = [s.name for s in specs if s.name not in tensors and all(s.name != w[0] for w in wrong)]
    if missing or unexpected or wrong:
        raise WeightError(folder, missing, sorted(unexpected), wrong)
    return tensors


def load_model(folder: str | Path, dtype: torch.dtype | str = torch.bfloat16,
               device: torch.device | str = "cuda:0", max_positions: int | None = None) -> DecoderModel:
    """Build the model config.json names and fill it from the folder's safetensors."""
    if isinstance(dtype, str):
        dtype = resolve_dtype(dtype)
    device = torch.device(device)
    spec, _cfg = read_spec(folder)
    model = DecoderModel(spec, dtype, device)
    if max_positions is not None:
        model.limit_positions(max_positions)
    model.bind(load_tensors(folder, model.weight_specs(), dtype, device, spec.ignored_name_patterns))
    return model
