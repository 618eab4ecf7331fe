"""Binds checkpoint tensors to a model's parts by tensor name.

Files: every ``model*.safetensors`` of the folder (omniserve/models/qwen2_vl.py:42-44).  Names and
the prefix rule: omniserve/model/qwen2_llm.py:196-219 (``model.language_model.`` if present, else
``model.``); q/k/v and gate/up are concatenated along the output dimension in that order
(qwen2_llm.py:207-216).  Unlike the reference, which fails with a bare KeyError, every problem of
a checkpoint is collected and reported in one error: missing tensors, unexpected tensors and
tensors of the wrong shape.

Storage types: a 16-bit float tensor is kept in bfloat16 (float32 when the engine runs in 32-bit);
a tensor the file stores in 32-bit stays 32-bit; integer tables become int32.
"""

from __future__ import annotations

import os
from typing import Dict, List, Optional, Tuple

import torch

from ..models.decoder import DecoderModel


class WeightsError(ValueError):
    """A checkpoint that does not fit the model; lists everything that is wrong with it."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong_shape: List[Tuple[str, tuple, tuple]], other: Optional[List[str]] = None):
        self.missing, self.unexpected, self.wrong_shape, self.other = missing, unexpected, wrong_shape, other or []
        lines = [f"checkpoint {where} does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong_shape:
            lines.append(f"  wrong shapes ({len(wrong_shape)}): " + ", ".join(
                f"{n}: file has {list(got)}, model needs {list(want)}" for n, got, want in wrong_shape))
        for o in self.other:
            lines.append("  " + o)
        super().__init__("\n".join(lines))


_FLOAT16 = (torch.bfloat16, torch.float16)
_FLOAT_WIDE = (torch.float32, torch.float64)
_ST_DTYPES = {"F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
              "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
              "BOOL": torch.bool}


def target_dtype(stored: torch.dtype, kind: str, engine_dtype: torch.dtype) -> torch.dtype:
    if kind == "int":
        return torch.int32
    if engine_dtype == torch.float32 or stored in _FLOAT_WIDE:
        return torch.float32
    return torch.bfloat16


class _Files:
    """Name -> (open file, shape, dtype) over all safetensors files of a folder."""

    def __init__(self, model_dir: str):
        from safetensors import safe_open
        self.handles = []
        self.index: Dict[str, int] = {}
        names = sorted(f for f in os.listdir(model_dir) if f.startswith("model") and f.endswith(".safetensors"))
        if not names:
            raise WeightsError(model_dir, [], [], [], ["no model*.safetensors file in the folder"])
        for fn in names:
            try:
                h = safe_open(os.path.join(model_dir, fn), framework="pt", device="cpu")
            except Exception as e:  # malformed file
                raise WeightsError(model_dir, [], [], [], [f"{fn}: not a readable safetensors file ({e})"]) from e
            self.handles.append(h)
            for k in h.keys():
                self.index[k] = len(self.handles) - 1

    def names(self) -> List[str]:
        return list(self.index)

    def meta(self, name: str) -> Tuple[tuple, torch.dtype]:
        sl = self.handles[self.index[name]].get_slice(name)
        return tuple(sl.get_shape()), _ST_DTYPES.get(sl.get_dtype(), torch.float32)

    def get(self, name: str) -> torch.Tensor:
        return self.handles[self.index[name]].get_tensor(name)


def expected_tensors(model: DecoderModel, decoder_prefix: str) -> List[Tuple[object, object, List[str]]]:
    """(part, ParamSpec, full checkpoint names of its sources) for every tensor of the model."""
    out = []
    for part, absolute in model.parts():
        base = "" if absolute else decoder_prefix
        for ps in part.param_specs():
            out.append((part, ps, [base + part.prefix + s for s in ps.sources]))
    return out


def detect_prefix(model: DecoderModel, names) -> str:
    probe = model.spec.embed_prefix + "weight"
    for p in model.spec.decoder_prefixes:
        if p + probe in names:
            return p
    return model.spec.decoder_prefixes[-1]


def load_weights(model: DecoderModel, model_dir: str, engine_dtype: torch.dtype, device) -> Dict[str, torch.dtype]:
    """Reads the folder's tensors into the model's parts on ``device``; returns name -> dtype kept."""
    files = _Files(model_dir)
    names = set(files.names())
    prefix = detect_prefix(model, names)
    expected = expected_tensors(model, prefix)
    missing: List[str] = []
    wrong: List[Tuple[str, tuple, tuple]] = []
    used = set()
    for _part, ps, full in expected:
        for n, shape in zip(full, ps.shapes):
            if n not in names:
                missing.append(n)
                continue
            used.add(n)
            got, _ = files.meta(n)
            if tuple(got) != tuple(shape):
                wrong.append((n, tuple(got), tuple(shape)))
    spec = model.spec
    unexpected = []
    for n in sorted(names - used):
        if n.startswith(spec.ignored_prefixes) or n.endswith(spec.ignored_suffixes):
            continue
        if spec.tie_word_embeddings and n == spec.head_prefix + "weight":
            continue  # a tied head stored a second time
        unexpected.append(n)
    if missing or wrong or unexpected:
        raise WeightsError(model_dir, sorted(missing), unexpected, wrong)

    kept: Dict[str, torch.dtype] = {}
    by_part: Dict[int, Tuple[object, Dict[str, torch.Tensor]]] = {}
    for part, ps, full in expected:
        stored = [files.meta(n)[1] for n in full]
        dt = target_dtype(stored[0], ps.kind, engine_dtype)
        for s in stored[1:]:
            if target_dtype(s, ps.kind, engine_dtype) == torch.float32 and ps.kind != "int":
                dt = torch.float32
        dest = torch.empty(ps.shape, dtype=dt, device=device)
        row = 0
        for n, shape in zip(full, ps.shapes):
            t = files.get(n)
            dest[row:row + shape[0]].copy_(t.to(dt) if t.dtype != dt else t)
            row += shape[0]
            kept[n] = dt
        by_part.setdefault(id(part), (part, {}))[1][ps.attr] = dest
    for part, tensors in by_part.values():
        part.bind(tensors)
    return kept
