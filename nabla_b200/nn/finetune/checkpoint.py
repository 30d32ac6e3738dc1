"""Fine-tuning checkpoints (reference: nabla/nn/finetune/checkpoint.py:19-170).

Format (kept byte-compatible in structure): a directory with ``tensors.npz``
(``np.savez_compressed`` of gathered host arrays named ``lora.<path>``, ``opt_m.<path>``,
``opt_v.<path>``; dict keys in sorted order, sequence items as ``[i]``) and ``meta.json``
(indent 2, sorted keys: ``step``, ``has_optimizer``, ``user_metadata``, ``tensor_keys``).
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any

import numpy as np

from ...core.common.pytree import is_tensor
from ...core.tensor.api import Tensor


def _collect(tree: Any, prefix: str, out: list[tuple[str, Tensor]]) -> None:
    if is_tensor(tree):
        out.append((prefix, tree))
    elif isinstance(tree, dict):
        for k in sorted(tree.keys(), key=str):
            _collect(tree[k], f"{prefix}.{k}" if prefix else str(k), out)
    elif isinstance(tree, (list, tuple)):
        for i, v in enumerate(tree):
            _collect(v, f"{prefix}[{i}]" if prefix else f"[{i}]", out)


def _assign(tree: Any, path: str, value: Tensor) -> Any:
    if path == "":
        return value
    if path.startswith("["):
        close = path.index("]")
        idx = int(path[1:close])
        rest = path[close + 1:]
        if rest.startswith("."):
            rest = rest[1:]
        if isinstance(tree, tuple):
            items = list(tree)
            items[idx] = _assign(items[idx], rest, value)
            return tuple(items)
        if isinstance(tree, list):
            tree[idx] = _assign(tree[idx], rest, value)
            return tree
        raise TypeError(f"Cannot assign index path {path} into {type(tree)}")
    # the key runs up to the next '.' or '['
    cut = len(path)
    for ch in (".", "["):
        p = path.find(ch)
        if p != -1:
            cut = min(cut, p)
    head, rest = path[:cut], path[cut:]
    if rest.startswith("."):
        rest = rest[1:]
    if not isinstance(tree, dict):
        raise TypeError(f"Cannot assign key path {path} into {type(tree)}")
    key: Any = head
    if head not in tree:
        try:
            key = int(head)
        except ValueError:
            key = head
    tree[key] = _assign(tree[key], rest, value)
    return tree


def _to_host(t: Tensor) -> np.ndarray:
    from ...types import DType

    if t.dtype is DType.bfloat16:
        return t.to(DType.float32).to_numpy()
    return t.to_numpy()


def save_finetune_checkpoint(path, *, lora_params: Any, optimizer_state: dict[str, Any] | None = None,
                             metadata: dict[str, Any] | None = None) -> None:
    out_dir = Path(path)
    out_dir.mkdir(parents=True, exist_ok=True)
    tensors: list[tuple[str, Tensor]] = []
    _collect(lora_params, "lora", tensors)
    step = None
    if optimizer_state is not None:
        s = optimizer_state.get("step", 0)
        step = int(s.item()) if is_tensor(s) else int(s)
        if "m" in optimizer_state:
            _collect(optimizer_state["m"], "opt_m", tensors)
        if "v" in optimizer_state:
            _collect(optimizer_state["v"], "opt_v", tensors)
    payload = {name: _to_host(t) for name, t in tensors}
    # write-then-rename so a crash never leaves a half-written checkpoint behind
    tmp = out_dir / "tensors.npz.tmp.npz"
    np.savez_compressed(tmp, **payload)
    os.replace(tmp, out_dir / "tensors.npz")
    meta = {"step": step, "has_optimizer": optimizer_state is not None, "user_metadata": metadata or {},
            "tensor_keys": sorted(payload.keys())}
    tmpm = out_dir / "meta.json.tmp"
    with tmpm.open("w", encoding="utf-8") as f:
        json.dump(meta, f, indent=2, sort_keys=True)
    os.replace(tmpm, out_dir / "meta.json")


def _restore(arr: np.ndarray, template: Tensor) -> Tensor:
    import torch

    t = torch.from_numpy(np.ascontiguousarray(arr)).to(device=template.device.to_torch(),
                                                         dtype=template.dtype.to_torch())
    out = Tensor(buffers=[t])
    sp = template._impl.sharding
    if sp is not None:
        from ...ops.communication import shard

        out = shard(out, sp.mesh, [d.clone() for d in sp.dim_specs], replicated_axes=set(sp.replicated_axes))
    if template.requires_grad:
        out.requires_grad = True
    return out


def load_finetune_checkpoint(path, *, lora_template: Any, optimizer_template: dict[str, Any] | None = None
                             ) -> tuple[Any, dict[str, Any] | None, dict[str, Any]]:
    d = Path(path)
    tp, mp = d / "tensors.npz", d / "meta.json"
    if not tp.exists():
        raise FileNotFoundError(f"Missing checkpoint tensor file: {tp}")
    if not mp.exists():
        raise FileNotFoundError(f"Missing checkpoint metadata file: {mp}")
    with mp.open(encoding="utf-8") as f:
        meta = json.load(f)
    npz = np.load(tp, allow_pickle=False)
    lora = lora_template
    paths: list[tuple[str, Tensor]] = []
    _collect(lora_template, "lora", paths)
    for name, tmpl in paths:
        if name not in npz:
            raise KeyError(f"Missing tensor key in checkpoint: {name}")
        lora = _assign(lora, name[len("lora") + 1:], _restore(npz[name], tmpl))
    opt = None
    if optimizer_template is not None and meta.get("has_optimizer", False):
        opt = {"step": int(meta.get("step") or 0), "m": optimizer_template.get("m"), "v": optimizer_template.get("v")}
        for slot in ("m", "v"):
            sp: list[tuple[str, Tensor]] = []
            _collect(opt[slot], f"opt_{slot}", sp)
            for name, tmpl in sp:
                if name not in npz:
                    raise KeyError(f"Missing tensor key in checkpoint: {name}")
                opt[slot] = _assign(opt[slot], name[len(f"opt_{slot}") + 1:], _restore(npz[name], tmpl))
    return lora, opt, meta
