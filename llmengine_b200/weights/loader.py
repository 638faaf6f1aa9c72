"""Binding weights to a model by tensor name, from a model folder or from a seed.

The reference binds graph constants to file tensors by name and checks shape, dtype and
device on bind (src/io/gguf_weight_loader.cpp:195-240), but silently skips a constant that
the file lacks (:512-513), which only fails later inside a kernel.  Here the set of names
must match exactly: one error lists every missing tensor, every unexpected tensor and every
wrong shape.
"""
from __future__ import annotations

import hashlib
import json
import os
import sys
from typing import Callable, Dict, Iterable, Mapping, Optional

import torch

from ..parts.base import WeightSpec
from .safetensors_io import SafetensorsFile, open_model_files, write_safetensors


class WeightError(ValueError):
    """The weight file does not fit the model."""


def stored_dtype(spec: WeightSpec, file_dtype: torch.dtype, compute: torch.dtype) -> torch.dtype:
    """The type a tensor is kept in on the device.  32-bit engine: everything is widened to
    float32.  bfloat16 engine: matrices are bfloat16 (a 32-bit file matrix is rounded to nearest
    even); vectors stored in 32-bit stay 32-bit, 16-bit ones stay bfloat16 (float16 is widened);
    integer tables are int32."""
    if spec.role == "table":
        return torch.int32
    if compute == torch.float32:
        return torch.float32
    if spec.role == "matrix":
        return torch.bfloat16
    return torch.bfloat16 if file_dtype == torch.bfloat16 else torch.float32


def check_names_and_shapes(specs: Mapping[str, WeightSpec], found: Mapping[str, tuple],
                           ignorable: Iterable[str] = ()) -> None:
    missing = sorted(n for n in specs if n not in found)
    unexpected = sorted(n for n in found if n not in specs and n not in set(ignorable))
    wrong = sorted((n, tuple(found[n]), tuple(specs[n].shape)) for n in specs
                   if n in found and tuple(found[n]) != tuple(specs[n].shape))
    if not (missing or unexpected or wrong):
        return
    lines = ["the weight file does not fit the model:"]
    if missing:
        lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
    if unexpected:
        lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
    if wrong:
        lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(
            f"{n} is {list(got)}, expected {list(want)}" for n, got, want in wrong))
    raise WeightError("\n".join(lines))


def load_model_weights(model, config, model_dir: str, compute: torch.dtype, device: torch.device) -> None:
    """Read every tensor the model declares from the folder's safetensors file(s)."""
    files = open_model_files(model_dir)
    canonical = getattr(config, "canonical_tensor_name", lambda n: n)
    where: Dict[str, tuple] = {}
    for f in files:
        for raw in f.names():
            name = canonical(raw)
            if name in where:
                raise WeightError(f"tensor {name!r} appears twice in {model_dir} (as {where[name][1]!r} and {raw!r})")
            where[name] = (f, raw)
    specs = model.weight_specs()
    # a tensor that a part shares with another part (a tied head) is sometimes stored all the same, as a copy
    ignorable = [n for n in model.tied_tensors() if n in where and n not in specs]
    for n in ignorable:
        print(f"[llmengine_b200] {n} is tied to {model.tied_tensors()[n]}: the file's copy is ignored", file=sys.stderr)
    check_names_and_shapes(specs, {n: f.shape(raw) for n, (f, raw) in where.items()}, ignorable)
    tensors: Dict[str, torch.Tensor] = {}
    for name, spec in specs.items():
        f, raw = where[name]
        t = f.tensor(raw)
        tensors[name] = t.to(device=device, dtype=stored_dtype(spec, t.dtype, compute), copy=True)
    model.load_weights(tensors)


# ----------------------------------------------------------------------------- random weights
def _tensor_seed(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little") & (2**63 - 1)


def _signed(c: int) -> int:
    return c - (1 << 64) if c >= (1 << 63) else c


_GAMMA, _M1, _M2 = _signed(0x9E3779B97F4A7C15), _signed(0xBF58476D1CE4E5B9), _signed(0x94D049BB133111EB)


def _mix64(z: torch.Tensor) -> torch.Tensor:
    """The splitmix64 finaliser on int64 tensors (products wrap modulo 2^64; shifts are made logical by masking)."""
    z = (z ^ ((z >> 30) & ((1 << 34) - 1))) * _M1
    z = (z ^ ((z >> 27) & ((1 << 37) - 1))) * _M2
    return z ^ ((z >> 31) & ((1 << 33) - 1))


def counter_normal(key: int, start: int, count: int, device: torch.device) -> torch.Tensor:
    """Elements start..start+count-1 of the stream of `key`: 32-bit variates with mean 0 and variance 1, each
    a function of (key, element index) alone.  An element is the sum of twelve 16-bit uniform integers cut from
    three hashes of its counter, centred: integer arithmetic until the last step, so every device, library
    version and chunking gives the same bits.  (The sum of twelve uniforms is the classic stand-in for a normal
    variate: right mean, variance and symmetry, tails that end at six standard deviations.)"""
    idx = torch.arange(start, start + count, dtype=torch.int64, device=device)
    base = idx * _GAMMA + _signed(key & ((1 << 64) - 1))
    total = torch.zeros(count, dtype=torch.int64, device=device)
    for j in range(3):
        h = _mix64(base + _signed((0xD1B54A32D192ED03 * (j + 1)) & ((1 << 64) - 1)))
        for k in range(4):
            total += (h >> (16 * k)) & 0xFFFF
    # 12 uniforms on {0..65535}: mean 12 * 32767.5 = 393210, variance 12 * (65536^2 - 1) / 12 ~ 65536^2
    return (total - 393210).to(torch.float32) * (1.0 / 65536.0)


def random_tensor(name: str, spec: WeightSpec, seed: int, device: torch.device = torch.device("cpu")) -> torch.Tensor:
    """A 32-bit tensor drawn from (seed, name, element index) alone, so that its values depend neither on the
    order of generation nor on the device that makes them: "normal" ~ N(0, 0.02), "gain" ~ 1 + N(0, 0.1)."""
    numel = 1
    for d in spec.shape:
        numel *= int(d)
    key = _tensor_seed(seed, name)
    out = torch.empty(numel, dtype=torch.float32, device=device)
    step = 1 << 24                                         # bounded temporaries for the large tables
    for a in range(0, numel, step):
        n = min(step, numel - a)
        out[a:a + n] = counter_normal(key, a, n, device)
    out = out.view(tuple(spec.shape))
    if spec.init == "gain":
        return 1.0 + 0.1 * out
    if spec.init == "normal":
        return 0.02 * out
    raise ValueError(f"tensor {name!r}: unknown init {spec.init!r}")


def random_model_weights(model, seed: int, compute: torch.dtype, device: torch.device,
                         file_dtype: torch.dtype = torch.bfloat16) -> None:
    """Fill a model with random weights directly on the device (no folder is written): the tensors that
    `write_random_model` would store for the same seed, bit for bit.  Values pass through `file_dtype` as
    they would through a file.  Where the kernel set has the generator (`random_fill`), every tensor is made
    by one launch straight into its stored type."""
    fill = getattr(model.rt.ops, "random_fill", None)
    tensors = {}
    for name, spec in model.weight_specs().items():
        stored = stored_dtype(spec, file_dtype, compute)
        if fill is not None and stored in (torch.float32, torch.bfloat16) and spec.init in ("normal", "gain"):
            t = torch.empty(tuple(spec.shape), dtype=stored, device=device)
            scale, offset = (0.02, 0.0) if spec.init == "normal" else (0.1, 1.0)
            tensors[name] = fill(t, _tensor_seed(seed, name), 0, scale, offset,
                                 round_bf16_first=file_dtype == torch.bfloat16 and stored != torch.bfloat16)
        else:
            t = random_tensor(name, spec, seed, device).to(file_dtype)
            tensors[name] = t.to(stored)
    model.load_weights(tensors)


def write_random_model(config, seed: int, out_dir: str, dtype: str = "bfloat16", shard_bytes: int = 0,
                       device: str = "cpu") -> str:
    """Random-weights mode: write `config.json` and `model.safetensors` for a configuration and a seed.
    `shard_bytes` > 0 writes `model-0000i-of-0000n.safetensors` files of about that size with a
    `model.safetensors.index.json` instead, as large checkpoints are laid out.  `device`: where the values
    are computed (they are the same everywhere; a GPU is only faster for large tables)."""
    from ..engine.model import Model
    from ..parts.base import Runtime

    file_dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    os.makedirs(out_dir, exist_ok=True)
    model = Model(config.model_spec(), Runtime(None, torch.device("cpu"), torch.float32, 1))
    dev = torch.device(device)
    tensors = {n: random_tensor(n, s, seed, dev).to(file_dtype).cpu() for n, s in model.weight_specs().items()}
    d = config.to_dict()
    d["torch_dtype"] = dtype
    with open(os.path.join(out_dir, "config.json"), "w", encoding="utf-8") as f:
        json.dump(d, f, indent=2)
    meta = {"format": "pt", "seed": str(seed)}
    if shard_bytes <= 0:
        write_safetensors(os.path.join(out_dir, "model.safetensors"), tensors, meta)
        return out_dir
    shards, size = [[]], 0
    for n in sorted(tensors):
        b = tensors[n].numel() * tensors[n].element_size()
        if shards[-1] and size + b > shard_bytes:
            shards.append([])
            size = 0
        shards[-1].append(n)
        size += b
    weight_map, total = {}, 0
    for i, names in enumerate(shards):
        fn = f"model-{i + 1:05d}-of-{len(shards):05d}.safetensors"
        write_safetensors(os.path.join(out_dir, fn), {n: tensors[n] for n in names}, meta)
        for n in names:
            weight_map[n] = fn
            total += tensors[n].numel() * tensors[n].element_size()
    with open(os.path.join(out_dir, "model.safetensors.index.json"), "w", encoding="utf-8") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=2)
    return out_dir
