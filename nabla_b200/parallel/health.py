"""Host-side peer liveness over the rendezvous store.

A rank that stops between two steps announces it (``announce_exit``); ranks that are still
running look at the store before their next launch (``check_peers``) and get a ``PeerLostError``
instead of entering a collective that can never complete. Heartbeats cover ranks that die
without announcing: ``beat()`` once per step, ``check_peers(max_silence_s=...)`` flags a rank
whose last beat is too old. Nothing here touches the GPU, so a lost peer never leaves kernels
or collectives of the survivors waiting on the device.

The reference has no failure detection (its multi-device path is single-process simulation);
this is the one-process-per-GPU counterpart of its checkpoint/resume story
(nabla/nn/finetune/checkpoint.py): detect on the host, stop cleanly, resume from a checkpoint.
"""
from __future__ import annotations

import time

import torch.distributed as dist


class PeerLostError(RuntimeError):
    def __init__(self, ranks, reason: str):
        super().__init__(f"rank(s) {sorted(ranks)} {reason}")
        self.ranks = sorted(ranks)


_store = None


def _get_store():
    global _store
    if _store is None:
        if not (dist.is_available() and dist.is_initialized()):
            return None
        from torch.distributed.distributed_c10d import _get_default_store

        _store = dist.PrefixStore("nabla_b200_health", _get_default_store())
    return _store


def reset() -> None:
    global _store
    _store = None


def announce_exit(reason: str = "left") -> None:
    """Tell the other ranks that this rank will take part in no further collective."""
    st = _get_store()
    if st is not None:
        st.set(f"gone/{dist.get_rank()}", reason)


def beat() -> None:
    """Record that this rank is alive (call once per step)."""
    st = _get_store()
    if st is not None:
        st.set(f"beat/{dist.get_rank()}", repr(time.time()))


def check_peers(max_silence_s: float | None = None) -> None:
    """Raise ``PeerLostError`` if a rank announced its exit, or (with ``max_silence_s``) if a
    rank that has beaten before has been silent for longer than that."""
    st = _get_store()
    if st is None:
        return
    world, me = dist.get_world_size(), dist.get_rank()
    gone, silent = [], []
    now = time.time()
    for r in range(world):
        if r == me:
            continue
        if st.check([f"gone/{r}"]):
            gone.append(r)
        elif max_silence_s is not None and st.check([f"beat/{r}"]):
            if now - float(st.get(f"beat/{r}").decode()) > max_silence_s:
                silent.append(r)
    if gone:
        raise PeerLostError(gone, "announced that they left")
    if silent:
        raise PeerLostError(silent, f"sent no heartbeat for more than {max_silence_s} s")
