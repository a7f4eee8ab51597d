# SPDX-License-Identifier: Apache-2.0
"""Hugging Face checkpoint layout: name mapping between the native fused parameters and HF tensors,
and safetensors reading / sharded writing.

Native ``qkv_proj`` = rows of ``q_proj``, ``k_proj``, ``v_proj`` stacked; native ``gate_up_proj`` = rows of
``gate_proj`` / ``up_proj`` interleaved in blocks of 64.  Everything else keeps its HF name.  The
directory layout written here (``config.json``, ``model.safetensors`` or
``model-0000i-of-0000N.safetensors`` + ``model.safetensors.index.json``, metadata ``{"format": "pt"}``)
is what arctic_training/checkpoint/hf_engine.py:73-154 produces and what ``transformers`` / vLLM load.
"""

from __future__ import annotations

import json
import re
from pathlib import Path
from typing import Callable
from typing import Dict
from typing import Iterable
from typing import Iterator
from typing import List
from typing import Optional
from typing import Tuple

import torch

from ..ops import reference as ref
from .arch import ArchConfig

_QKV = re.compile(r"^(.*self_attn\.)qkv_proj\.(weight|bias)$")
_GU = re.compile(r"^(.*)gate_up_proj\.weight$")


def native_to_hf(name: str, tensor: torch.Tensor, cfg: ArchConfig) -> List[Tuple[str, torch.Tensor]]:
    """Expand one native parameter into the HF tensors it corresponds to."""
    for conv in _EXTRA_NATIVE_TO_HF:
        res = conv(name, tensor, cfg)
        if res is not None:
            return res
    m = _QKV.match(name)
    if m:
        hq = cfg["num_attention_heads"]
        hkv = cfg.get("num_key_value_heads") or hq
        d = cfg.head_dim_
        q, k, v = tensor.split([hq * d, hkv * d, hkv * d], dim=0)
        pre, kind = m.group(1), m.group(2)
        return [(f"{pre}q_proj.{kind}", q), (f"{pre}k_proj.{kind}", k), (f"{pre}v_proj.{kind}", v)]
    m = _GU.match(name)
    if m and tensor.dim() == 2:
        g, u = ref.deinterleave_gate_up_rows(tensor)
        return [(f"{m.group(1)}gate_proj.weight", g), (f"{m.group(1)}up_proj.weight", u)]
    return [(name, tensor)]


def hf_to_native_state_dict(hf: Dict[str, torch.Tensor], cfg: ArchConfig) -> Dict[str, torch.Tensor]:
    """Fold an HF state dict into native fused parameters."""
    out: Dict[str, torch.Tensor] = {}
    hf = dict(hf)
    for conv in _EXTRA_HF_TO_NATIVE:
        conv(hf, out, cfg)
    for name in sorted(hf):
        if name not in hf:
            continue
        if name.endswith("self_attn.q_proj.weight") or name.endswith("self_attn.q_proj.bias"):
            pre, kind = name.rsplit("q_proj.", 1)
            parts = [hf[f"{pre}{x}_proj.{kind}"] for x in ("q", "k", "v")]
            out[f"{pre}qkv_proj.{kind}"] = torch.cat(parts, dim=0)
        elif re.search(r"self_attn\.[kv]_proj\.(weight|bias)$", name):
            continue
        elif name.endswith("mlp.gate_proj.weight") or name.endswith("shared_expert.gate_proj.weight"):
            pre = name[: -len("gate_proj.weight")]
            out[f"{pre}gate_up_proj.weight"] = ref.interleave_gate_up_rows(hf[name], hf[f"{pre}up_proj.weight"])
        elif name.endswith("mlp.up_proj.weight") or name.endswith("shared_expert.up_proj.weight"):
            continue
        else:
            out[name] = hf[name]
    return out


# model families with extra fused tensors (MoE experts) register converters here
_EXTRA_NATIVE_TO_HF: List[Callable] = []
_EXTRA_HF_TO_NATIVE: List[Callable] = []


def iter_hf_tensors(named: Iterable[Tuple[str, torch.Tensor]], cfg: ArchConfig) -> Iterator[Tuple[str, torch.Tensor]]:
    for name, t in named:
        for item in native_to_hf(name, t, cfg):
            yield item


def read_safetensors_dir(path: Path) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    path = Path(path)
    index = path / "model.safetensors.index.json"
    tensors: Dict[str, torch.Tensor] = {}
    if index.exists():
        with open(index) as fh:
            files = sorted(set(json.load(fh)["weight_map"].values()))
    elif (path / "model.safetensors").exists():
        files = ["model.safetensors"]
    else:
        files = sorted(p.name for p in path.glob("*.safetensors"))
    for f in files:
        tensors.update(load_file(str(path / f)))
    if not tensors and (path / "pytorch_model.bin").exists():
        tensors = torch.load(path / "pytorch_model.bin", map_location="cpu", weights_only=True)
    return tensors


class ShardedSafetensorsWriter:
    """Streams tensors into ``model-0000i-of-0000N.safetensors`` shards of bounded size and writes the
    index at the end; a single shard is renamed to ``model.safetensors``."""

    def __init__(self, out_dir: Path, max_shard_bytes: int = 4 << 30) -> None:
        self.out_dir = Path(out_dir)
        self.out_dir.mkdir(parents=True, exist_ok=True)
        self.max_shard_bytes = max_shard_bytes
        self._cur: Dict[str, torch.Tensor] = {}
        self._cur_bytes = 0
        self._shards: List[List[str]] = []
        self._tmp_files: List[Path] = []
        self.total_bytes = 0
        self.total_params = 0

    def add(self, name: str, tensor: torch.Tensor) -> None:
        t = tensor.detach().to("cpu").contiguous().clone()
        nbytes = t.numel() * t.element_size()
        if self._cur and self._cur_bytes + nbytes > self.max_shard_bytes:
            self._flush()
        self._cur[name] = t
        self._cur_bytes += nbytes
        self.total_bytes += nbytes
        self.total_params += t.numel()

    def _flush(self) -> None:
        from safetensors.torch import save_file

        if not self._cur:
            return
        tmp = self.out_dir / f"model-tmp-{len(self._tmp_files):05d}.safetensors"
        save_file(self._cur, str(tmp), metadata={"format": "pt"})
        self._tmp_files.append(tmp)
        self._shards.append(list(self._cur))
        self._cur, self._cur_bytes = {}, 0

    def finish(self) -> None:
        self._flush()
        n = len(self._tmp_files)
        if n == 1:
            self._tmp_files[0].rename(self.out_dir / "model.safetensors")
            return
        weight_map = {}
        for i, (tmp, names) in enumerate(zip(self._tmp_files, self._shards), start=1):
            fname = f"model-{i:05d}-of-{n:05d}.safetensors"
            tmp.rename(self.out_dir / fname)
            for k in names:
                weight_map[k] = fname
        with open(self.out_dir / "model.safetensors.index.json", "w") as fh:
            json.dump({"metadata": {"total_size": self.total_bytes}, "weight_map": weight_map}, fh, indent=2)


def save_config(cfg: ArchConfig, out_dir: Path, dtype: Optional[torch.dtype] = None) -> None:
    d = cfg.to_json_dict()
    if dtype is not None:
        d["torch_dtype"] = str(dtype).replace("torch.", "")
    with open(Path(out_dir) / "config.json", "w") as fh:
        json.dump(d, fh, indent=2, sort_keys=True)


def load_pretrained_into(model: torch.nn.Module, path: Path, cfg: ArchConfig, strict: bool = True) -> None:
    """Load an HF-layout checkpoint directory into a native model (fusing projections on the fly)."""
    hf = read_safetensors_dir(Path(path))
    if not hf:
        raise FileNotFoundError(f"no weights found under {path}")
    native = hf_to_native_state_dict(hf, cfg)
    own = dict(model.named_parameters())
    own.update(dict(model.named_buffers()))
    missing = [k for k in own if k not in native and not (k == "lm_head.weight" and cfg.get("tie_word_embeddings"))]
    unexpected = [k for k in native if k not in own]
    if strict and (missing or unexpected):
        raise KeyError(f"checkpoint mismatch: missing={missing[:8]} unexpected={unexpected[:8]}")
    with torch.no_grad():
        for k, t in native.items():
            if k in own:
                dst = own[k]
                if getattr(dst, "_num_experts", 0) and t.shape[0] == dst._num_experts != dst.shape[0]:
                    t = t[dst._first_expert : dst._first_expert + dst.shape[0]]  # this rank's experts only
                dst.copy_(t.to(dst.dtype))
