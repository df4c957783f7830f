"""Loads the tensors a model asks for, by name, and says everything that is wrong at once.

Stored precision is kept: BF16 stays bfloat16, F32 stays float32 (F16 is widened to float32, so no
bit is lost), integer tables become int32. What the runtime's mode needs is decided later by the
parts (`Runtime.matrix`, `Runtime.vector`). The reference names one problem per error
("{name} is not in the checkpoint", "{name} has shape [...], expected [...]":
crates/specrt/src/weights.rs:258-273, 377-401); here one `WeightError` lists all missing and
unexpected tensors and all wrong shapes.

A checkpoint's own names are mapped to the model's names first:
  * rename rules, `{part of a name: its replacement}`, applied to every stored name in the order of
    the mapping's keys (crates/specrt/src/weights.rs:226-240; a model spec's `[tensors]` table);
  * the decoder's root: a checkpoint that keeps the decoder under `model.language_model.` or
    `language_model.model.` instead of `model.` (a text model saved inside a larger one) is read
    as if it were stored under `model.` (crates/specrt/src/weights.rs:365-375).

Tensors are checked from the file headers alone, then read one part at a time (`stream_into`), so
the device never holds more than the bound model plus the sources of one part; the reference
uploads in plan order for the same reason (crates/specrt/src/runtime.rs:35-67, 184-287).
"""
from __future__ import annotations

import sys
from collections import Counter
from typing import Iterable, Mapping, Optional

import torch

from ..parts.base import WeightSpec
from .safetensors_io import Checkpoint, CheckpointError

ALTERNATIVE_ROOTS = ("model.language_model", "language_model.model")


class WeightError(ValueError):
    """The checkpoint does not hold exactly the tensors the model reads."""

    def __init__(self, missing, unexpected, wrong_shape, other=()):
        self.missing, self.unexpected, self.wrong_shape, self.other = list(missing), list(unexpected), list(wrong_shape), list(other)
        lines = ["the checkpoint does not match the model:"]
        if self.missing:
            lines.append(f"  missing tensors ({len(self.missing)}): " + ", ".join(self.missing))
        if self.unexpected:
            lines.append(f"  unexpected tensors ({len(self.unexpected)}): " + ", ".join(self.unexpected))
        for name, got, want in self.wrong_shape:
            lines.append(f"  {name} has shape {list(got)}, expected {list(want)}")
        lines += [f"  {o}" for o in self.other]
        super().__init__("\n".join(lines))


def _as_stored(t: torch.Tensor, role: str) -> torch.Tensor:
    if role == "table":
        return t.to(torch.int32)
    if t.dtype == torch.float16:
        return t.to(torch.float32)
    return t


def public_names(stored: Iterable[str], wanted: Iterable[str], rules: Optional[Mapping[str, str]] = None, root: str = "model") -> dict[str, str]:
    """{the model's name: the checkpoint's name} for every stored tensor, after the rename rules and
    the probing of the decoder's root. Two stored names that end up under one public name are an error."""
    stored = list(stored)
    renamed: dict[str, str] = {}
    for name in stored:
        public = name
        for old, new in sorted((rules or {}).items()):
            public = public.replace(old, new)
        if public in renamed:
            raise CheckpointError(f"tensors {renamed[public]} and {name} are both renamed to {public}")
        renamed[public] = name
    probe = next((w for w in wanted if w.startswith(root + ".")), None)
    if probe is not None and probe not in renamed:
        for alt in ALTERNATIVE_ROOTS:
            if alt + probe[len(root):] in renamed:
                moved: dict[str, str] = {}
                for public, name in renamed.items():
                    if public.startswith(alt + "."):
                        public = root + public[len(alt):]
                    if public in moved:
                        raise CheckpointError(f"tensors {moved[public]} and {name} both stand for {public}")
                    moved[public] = name
                return moved
    return renamed


class WeightStore:
    """A model folder's checkpoint seen through the model's tensor names, checked against the
    model's wants when it is opened. `unexpected` lists the stored tensors the model does not read."""

    def __init__(self, model_dir, specs: Iterable[WeightSpec], ignored: Iterable[str] = (), rules: Optional[Mapping[str, str]] = None,
                 root: str = "model", strict: bool = True):
        self.specs = {s.name: s for s in specs}
        self.ckpt = Checkpoint(model_dir)
        try:
            self.names = public_names(self.ckpt.names(), self.specs, rules, root)
            self._check(set(ignored), strict)
        except Exception:
            self.ckpt.close()
            raise

    def _check(self, ignored: set, strict: bool) -> None:
        wanted, have = self.specs, set(self.names)
        info = {n: self.ckpt.tensors[self.names[n]] for n in have}
        missing = sorted(set(wanted) - have)
        self.unexpected = sorted(have - set(wanted) - ignored)
        wrong = [(n, info[n].shape, wanted[n].shape) for n in sorted(set(wanted) & have) if tuple(info[n].shape) != tuple(wanted[n].shape)]
        other = []
        for n in sorted(set(wanted) & have):
            dt = info[n].dtype
            floating = dt in ("BF16", "F16", "F32")
            if wanted[n].role == "table" and dt not in ("I32", "I64"):
                other.append(f"{n} is stored as {dt}, expected an integer table")
            elif wanted[n].role != "table" and not floating:
                other.append(f"{n} is stored as {dt}, expected BF16, F16 or F32 (quantized formats are not read)")
        if missing or wrong or other or (strict and self.unexpected):
            raise WeightError(missing, self.unexpected, wrong, other)

    def read(self, name: str, device: Optional[torch.device] = None) -> torch.Tensor:
        t = _as_stored(self.ckpt.read(self.names[name]), self.specs[name].role)
        return t.to(device) if device is not None else t

    def close(self) -> None:
        self.ckpt.close()


def load_weights(model_dir, specs: Iterable[WeightSpec], ignored: Iterable[str] = (), device: Optional[torch.device] = None,
                 rules: Optional[Mapping[str, str]] = None, root: str = "model", strict: bool = True) -> dict[str, torch.Tensor]:
    """Every tensor the specs name, at once (tests and small models; the engine streams instead)."""
    store = WeightStore(model_dir, specs, ignored, rules, root, strict)
    try:
        return {name: store.read(name, device) for name in store.specs}
    finally:
        store.close()


class _Streamed:
    """What a part sees while it binds: `weights[name]` reads the tensor to the device at that moment.
    A tensor that several parts read (a tied embedding) is kept until the last of them has asked."""

    def __init__(self, store: WeightStore, device, users: Counter):
        self.store, self.device, self.users, self.kept = store, device, users, {}

    def __getitem__(self, name: str) -> torch.Tensor:
        if name not in self.store.specs:
            raise KeyError(f"{name} is not among the tensors the model declared (weight_specs)")
        t = self.kept.get(name)
        if t is None:
            t = self.store.read(name, self.device)
        self.users[name] -= 1
        if self.users[name] > 0:
            self.kept[name] = t
        else:
            self.kept.pop(name, None)
        return t


def stream_into(decoder, rt, model_dir, rules: Optional[Mapping[str, str]] = None, strict: bool = False, say=None) -> list[str]:
    """Bind every part of `decoder` from the checkpoint in `model_dir`, one part at a time: a part's
    tensors are read to the device when its `bind` asks for them and dropped as soon as it returns.
    Returns the stored tensors the model did not read (an error instead when `strict`)."""
    plan = decoder.plan
    store = WeightStore(model_dir, decoder.weight_specs(), plan.ignored_tensors, rules, getattr(plan, "root", "model"), strict)
    try:
        users = Counter(s.name for p in decoder.parts() for s in p.weight_specs())
        weights = _Streamed(store, rt.device, users)
        decoder.rt = rt
        for part in decoder.parts():
            part.bind(weights, rt)
        if store.unexpected and say is not False:
            (say or (lambda m: print(m, file=sys.stderr)))(
                f"[inference_bench_b200] {len(store.unexpected)} tensor(s) of the checkpoint are not read by this model: "
                + ", ".join(store.unexpected[:8]) + (" ..." if len(store.unexpected) > 8 else ""))
        return store.unexpected
    finally:
        store.close()


__all__ = ["load_weights", "stream_into", "public_names", "WeightStore", "WeightError", "CheckpointError"]
