"""Weights by tensor name from a model folder, checked against what the model
expects, with one error that lists everything wrong.

The reference names the missing tensor and stops at the first
(crates/ai-engine-runtime/src/loader.rs:62,65; arch/model.rs:138-144); here the
folder is compared with the model's whole list first, so one message names all
missing tensors, all unexpected ones and all wrong shapes.

Dtype policy: compute dtype bfloat16 keeps bf16 as stored, turns f16 into
bf16, and leaves a tensor stored in 32-bit as it is; integer tables (a spec
with `init="int"`) become int32.  Compute dtype float32 widens every floating
tensor to f32 (loader.rs:733-744 does the same widening).  A weight stored as
integers where the model wants floating point (a quantised file) is refused in
the same message, by name, as the reference refuses dtypes it does not take
(loader.rs:748).
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Sequence, Tuple

import torch

from .safetensors_io import SafetensorsError, SafetensorsFile


class WeightError(ValueError):
    """The folder's tensors do not fit the model."""


@dataclass(frozen=True)
class TensorSpec:
    """One tensor that a part wants: HF name, shape, how random weights fill it
    (`normal`: N(0, std); `ones`: 1 + N(0, norm_std); `int`: uniform ints below
    `high`), and `alternatives`: names that may stand in when it is absent (a
    tied head reads the embedding; an embedding absent from a tied file reads
    lm_head, crates/ai-engine-runtime/src/loader.rs:129-151)."""
    name: str
    shape: Tuple[int, ...]
    init: str = "normal"
    alternatives: Tuple[str, ...] = ()
    high: int = 0
    stored: bool = True     # False: never written by the random-weights mode (tied head)


def _storage_dtype(stored: torch.dtype, compute: torch.dtype) -> torch.dtype:
    if not stored.is_floating_point:
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if stored in (torch.float32, torch.float64):
        return torch.float32
    return torch.bfloat16


class ModelFolder:
    """All *.safetensors files of a folder as one name -> tensor map."""

    def __init__(self, model_dir: str):
        self.model_dir = model_dir
        if not os.path.isdir(model_dir):
            raise WeightError(f"{model_dir}: not a folder")
        names = sorted(f for f in os.listdir(model_dir) if f.endswith(".safetensors"))
        index = os.path.join(model_dir, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                wm = json.load(f).get("weight_map", {})
            listed = sorted(set(wm.values()))
            absent = [n for n in listed if n not in names]
            if absent:
                raise WeightError(f"{model_dir}: index names files that are absent: {absent}")
            names = listed
        if not names:
            raise WeightError(f"{model_dir}: no *.safetensors file")
        self.files: List[SafetensorsFile] = []
        self.where: Dict[str, SafetensorsFile] = {}
        try:
            for n in names:
                sf = SafetensorsFile(os.path.join(model_dir, n))
                self.files.append(sf)
                for t in sf.names():
                    self.where[t] = sf
        except SafetensorsError as e:
            raise WeightError(str(e)) from None

    def names(self) -> List[str]:
        return list(self.where)

    def info(self, name: str):
        return self.where[name].info(name)

    def tensor(self, name: str) -> torch.Tensor:
        return self.where[name].tensor(name)

    def close(self) -> None:
        for f in self.files:
            f.close()


def check_and_resolve(specs: Sequence[TensorSpec], available: Dict[str, Tuple[torch.dtype, tuple]],
                      where: str = "", ignored: Sequence[str] = ()) -> Dict[str, str]:
    """Map every wanted name to the stored name that provides it, or raise one
    WeightError listing missing tensors, unexpected tensors, wrong shapes and wrong
    dtypes.  `ignored`: name endings of stored tensors that are no parameters (buffers
    that some exporters write) and are passed over."""
    missing, wrong, wrong_dtype, resolved, used = [], [], [], {}, set()
    for s in specs:
        src = None
        for cand in (s.name,) + tuple(s.alternatives):
            if cand in available:
                src = cand
                break
        if src is None:
            alt = f" (nor {', '.join(s.alternatives)})" if s.alternatives else ""
            missing.append(f"{s.name}{alt} {list(s.shape)}")
            continue
        dt, shape = available[src]
        if tuple(shape) != tuple(s.shape):
            wrong.append(f"{src}: stored {list(shape)}, model wants {list(s.shape)}")
        if isinstance(dt, torch.dtype) and dt.is_floating_point == (s.init == "int"):
            want = "integers" if s.init == "int" else "floating point (F32, F16 or BF16)"
            wrong_dtype.append(f"{src}: stored as {str(dt).replace('torch.', '')}, model wants {want}")
        resolved[s.name] = src
        used.add(src)
    wanted_names = {s.name for s in specs} | {a for s in specs for a in s.alternatives}
    unexpected = sorted(n for n in available if n not in used and n not in wanted_names
                        and not any(n.endswith(e) for e in ignored))
    if missing or wrong or unexpected or wrong_dtype:
        parts = [f"weights{' in ' + where if where else ''} do not fit the model:"]
        if missing:
            parts.append(f"  missing tensors ({len(missing)}): " + "; ".join(missing))
        if unexpected:
            parts.append(f"  unexpected tensors ({len(unexpected)}): " + "; ".join(unexpected))
        if wrong:
            parts.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        if wrong_dtype:
            parts.append(f"  wrong dtypes ({len(wrong_dtype)}): " + "; ".join(wrong_dtype))
        raise WeightError("\n".join(parts))
    return resolved


class WeightSource:
    """What parts load from: `get(name)` returns the tensor on the device in its
    storage dtype.  Built from a folder (checked) or from a dict of tensors."""

    def __init__(self, fetch: Callable[[str], torch.Tensor], resolved: Dict[str, str],
                 compute_dtype: torch.dtype, device):
        self._fetch, self._resolved = fetch, resolved
        self.compute_dtype, self.device = compute_dtype, device
        self._on_device: Dict[str, torch.Tensor] = {}
        self._shared = None           # None: keep every tensor until release()

    def keep_only(self, names) -> None:
        """Name the tensors that more than one part reads (a tied head and its embedding): only these
        are kept until release(), so that both get one device copy.  Every other tensor belongs to the
        part that fetched it; what that part fuses into another tensor is then freed with the part's
        last reference, and loading never holds much more than the model itself."""
        self._shared = {self._resolved.get(n, n) for n in names}

    def get(self, name: str) -> torch.Tensor:
        src = self._resolved.get(name, name)
        t = self._on_device.get(src)
        if t is None:        # a tensor wanted twice (tied head) is uploaded once
            t = self._fetch(src)
            dt = _storage_dtype(t.dtype, self.compute_dtype)
            t = t.to(device=self.device, dtype=dt).contiguous()
            if self._shared is None or src in self._shared:
                self._on_device[src] = t
        return t

    def release(self) -> None:
        self._on_device.clear()


def open_folder(model_dir: str, specs: Sequence[TensorSpec], compute_dtype: torch.dtype,
                device, ignored: Sequence[str] = ()) -> Tuple[WeightSource, ModelFolder]:
    folder = ModelFolder(model_dir)
    available = {n: folder.info(n) for n in folder.names()}
    resolved = check_and_resolve(specs, available, where=model_dir, ignored=ignored)
    return WeightSource(folder.tensor, resolved, compute_dtype, device), folder


def from_tensors(tensors: Dict[str, torch.Tensor], specs: Sequence[TensorSpec],
                 compute_dtype: torch.dtype, device) -> WeightSource:
    available = {n: (t.dtype, tuple(t.shape)) for n, t in tensors.items()}
    resolved = check_and_resolve(specs, available, where="the given tensors")
    return WeightSource(tensors.__getitem__, resolved, compute_dtype, device)
