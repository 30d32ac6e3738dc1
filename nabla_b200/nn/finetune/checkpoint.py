"""Fine-tuning checkpoints (reference: nabla/nn/finetune/checkpoint.py:19-170).

On-disk format, the compatibility surface shared with the reference: a directory holding
``tensors.npz`` (``np.savez_compressed`` of gathered host arrays) and ``meta.json`` (indent 2,
sorted keys ``step``, ``has_optimizer``, ``user_metadata``, ``tensor_keys``). Array names are the
pytree path of the tensor under one of three roots: ``lora.<path>`` for the adapter tree,
``opt_m.<path>`` / ``opt_v.<path>`` for the AdamW moments; dict keys (sorted) join with ``.``,
sequence positions appear as ``[i]``.

Both directions work on flattened trees: the names come from the tree structure
(``pytree.leaf_names``), a load fills a list of leaves by name and unflattens it onto the
template's structure, so no path string is ever parsed.

One process per GPU: every rank takes part in the gather of sharded tensors (``to_numpy`` is
collective), rank 0 alone writes, to rank-private temporary names followed by an atomic rename, and
a barrier keeps every rank inside the call until the files are in place.
"""
from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any

import numpy as np

from ...core.common import pytree
from ...core.tensor.api import Tensor

_ROOTS = (("lora", None), ("opt_m", "m"), ("opt_v", "v"))


def _named_tensors(tree: Any, root: str) -> tuple[list[str], list, "pytree.PyTreeDef"]:
    leaves, td = pytree.tree_flatten(tree)
    return pytree.leaf_names(td, root), leaves, td


def _host_array(t: Tensor) -> np.ndarray:
    from ...types import DType

    # numpy has no bfloat16: those tensors are stored widened (exactly) to float32
    return (t.to(DType.float32) if t.dtype is DType.bfloat16 else t).to_numpy()


def _dist_rank_world() -> tuple[int, int]:
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
    except Exception:
        pass
    return 0, 1


def _publish(tmp: Path, final: Path) -> None:
    os.replace(tmp, final)          # atomic on one filesystem: readers see the old or the new file


def save_finetune_checkpoint(path, *, lora_params: Any, optimizer_state: dict[str, Any] | None = None,
                             metadata: dict[str, Any] | None = None) -> None:
    """Write ``tensors.npz`` + ``meta.json`` under ``path``. Call it on EVERY rank of a distributed
    run (sharded tensors are gathered collectively); only rank 0 touches the file system."""
    rank, world = _dist_rank_world()
    groups = [("lora", lora_params)]
    step = None
    if optimizer_state is not None:
        s = optimizer_state.get("step", 0)
        step = int(s.item()) if isinstance(s, Tensor) else int(s)
        groups += [(root, optimizer_state[slot]) for root, slot in _ROOTS[1:] if slot in optimizer_state]
    payload: dict[str, np.ndarray] = {}
    for root, tree in groups:
        names, leaves, _ = _named_tensors(tree, root)
        for name, leaf in zip(names, leaves):
            if isinstance(leaf, Tensor):
                payload[name] = _host_array(leaf)            # collective when the tensor is sharded
    if rank == 0:
        out_dir = Path(path)
        out_dir.mkdir(parents=True, exist_ok=True)
        tag = f"{os.getpid()}.r{rank}"
        tmp_t = out_dir / f".tensors.{tag}.tmp.npz"          # savez appends .npz to other suffixes
        np.savez_compressed(tmp_t, **payload)
        _publish(tmp_t, out_dir / "tensors.npz")
        meta = {"step": step, "has_optimizer": optimizer_state is not None, "user_metadata": metadata or {},
                "tensor_keys": sorted(payload)}
        tmp_m = out_dir / f".meta.{tag}.tmp"
        tmp_m.write_text(json.dumps(meta, indent=2, sort_keys=True), encoding="utf-8")
        _publish(tmp_m, out_dir / "meta.json")
    if world > 1:
        import torch.distributed as dist

        dist.barrier()              # nobody leaves (or exits) before the checkpoint is complete


def _like(template: Tensor, arr: np.ndarray) -> Tensor:
    """Host array -> tensor with the template's dtype, device, sharding and requires_grad."""
    import torch

    t = torch.from_numpy(np.ascontiguousarray(arr)).reshape(arr.shape).to(device=template.device.to_torch(), dtype=template.dtype.to_torch())
    out = Tensor(buffers=[t])
    sp = template._impl.sharding
    if sp is not None:
        from ...ops.communication import shard

        out = shard(out, sp.mesh, [d.clone() for d in sp.dim_specs], replicated_axes=set(sp.replicated_axes))
    if template.requires_grad:
        out.requires_grad = True
    return out


def _fill(template: Any, root: str, arrays) -> Any:
    names, leaves, td = _named_tensors(template, root)
    new = []
    for name, leaf in zip(names, leaves):
        if not isinstance(leaf, Tensor):
            new.append(leaf)
            continue
        if name not in arrays:
            raise KeyError(f"Missing tensor key in checkpoint: {name}")
        new.append(_like(leaf, arrays[name]))
    return pytree.tree_unflatten(td, new)


def load_finetune_checkpoint(path, *, lora_template: Any, optimizer_template: dict[str, Any] | None = None
                             ) -> tuple[Any, dict[str, Any] | None, dict[str, Any]]:
    """Returns ``(lora_params, optimizer_state | None, meta)``; the templates give structure, dtype,
    device and sharding of what is rebuilt. Every rank reads the files itself."""
    d = Path(path)
    for f in (d / "tensors.npz", d / "meta.json"):
        if not f.exists():
            kind = "tensor" if f.suffix == ".npz" else "metadata"
            raise FileNotFoundError(f"Missing checkpoint {kind} file: {f}")
    meta = json.loads((d / "meta.json").read_text(encoding="utf-8"))
    arrays = np.load(d / "tensors.npz", allow_pickle=False)
    lora = _fill(lora_template, "lora", arrays)
    opt = None
    if optimizer_template is not None and meta.get("has_optimizer", False):
        opt = {"step": int(meta.get("step") or 0)}
        for root, slot in _ROOTS[1:]:
            opt[slot] = _fill(optimizer_template.get(slot), root, arrays)
    return lora, opt, meta
