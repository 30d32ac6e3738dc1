"""Symmetric workspaces over NVLink peer memory and the native collective entry points.

One workspace per device group (= the ranks spanned by a set of mesh axes): the same
allocation on every GPU of the group, mapped into every peer and, where the fabric supports it,
bound to an NVSwitch multicast object (NVLS). torch's symmetric-memory allocator does the handle
exchange; the kernels that read and write the peers' memory are ours
(``csrc/peer_collectives.cu``, and the fused GEMM + all-reduce in ``csrc/gemm_tcgen05.cu``).

``NABLA_B200_COMM=nccl`` disables this path (NCCL baseline); ``NABLA_B200_NVLS=0`` keeps the
kernels on plain peer loads/stores (used by the failure-detection tests).
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

_workspaces: dict = {}
_lib = None
_enabled: bool | None = None
launch_count = 0
DEFAULT_BYTES = int(os.environ.get("NABLA_B200_SYMM_MB", "640")) * 1024 * 1024
CANARY_BYTES, CANARY_VALUE = 4096, 0xA5
c_int, c_ll, c_vp, c_uint, c_ull = ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_uint, ctypes.c_ulonglong


def _L():
    global _lib
    if _lib is None:
        from ..native import load

        lib = load("libnb_comm.so")
        lib.nb_comm_flag_bytes.restype = c_int
        lib.nb_comm_tile_flag_offset.restype = c_int
        lib.nb_comm_done_offset.restype = c_int
        lib.nb_comm_allreduce.restype = c_int
        lib.nb_comm_allreduce.argtypes = [c_vp, c_vp, c_int, c_int, c_vp, c_ll, c_vp, c_ll, c_int, c_int, c_int, c_int,
                                          c_vp, c_vp]
        lib.nb_comm_gather.restype = c_int
        lib.nb_comm_gather.argtypes = [c_vp, c_int, c_int, c_vp, c_ll, c_vp, c_ll, c_int, c_int, c_int, c_int, c_vp, c_vp]
        lib.nb_comm_barrier.restype = c_int
        lib.nb_comm_barrier.argtypes = [c_vp, c_int, c_int, c_vp, c_vp, c_vp]
        lib.nb_comm_adamw_reduce.restype = c_int
        lib.nb_comm_adamw_reduce.argtypes = ([c_vp, c_int, c_int, c_vp, c_vp, c_vp, c_ll, c_vp, c_vp, c_vp, c_ll] +
                                             [ctypes.c_float] * 8 + [c_vp, c_int, c_vp, c_vp])
        lib.nb_comm_permute.restype = c_int
        lib.nb_comm_permute.argtypes = [c_vp, c_int, c_int, c_vp, c_ll, c_vp, c_vp, c_ll, c_int, c_int, c_int, c_vp, c_vp]
        lib.nb_comm_wait_flag.restype = c_int
        lib.nb_comm_wait_flag.argtypes = [c_vp, c_uint, c_vp, c_ull, c_vp]
        _lib = lib
    return _lib


class Workspace:
    """Symmetric buffer of one device group plus its epoch counter."""

    def __init__(self, pg, ranks: list[int], nbytes: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.pg, self.ranks = pg, ranks
        self.world = len(ranks)
        self.rank = ranks.index(dist.get_rank())
        self.flag_bytes = _L().nb_comm_flag_bytes()
        self.nbytes = int(nbytes)
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        self.buf.zero_()
        self.hdl = symm_mem.rendezvous(self.buf, group=pg)
        self.ptrs_dev = int(self.hdl.buffer_ptrs_dev)
        use_nvls = os.environ.get("NABLA_B200_NVLS", "1") != "0"
        mc = 0
        try:
            mc = int(self.hdl.multicast_ptr) if use_nvls else 0
        except Exception:
            mc = 0
        self.mc_ptr = mc
        # device-side call counters: [0] collectives, [1] fused all-gathers, [2] fused done counts
        self.ctr = torch.zeros(8, dtype=torch.int32, device=self.buf.device)
        self.data = self.buf[self.flag_bytes:]
        self.data_bytes = self.nbytes - self.flag_bytes
        # guard bytes at the very end of the allocation: no kernel is ever given an extent that
        # reaches them (`supports`, the fused launchers' size checks), so `check_canary` finding
        # them changed means some kernel wrote past its region
        self.buf[-CANARY_BYTES:].fill_(CANARY_VALUE)
        torch.cuda.synchronize()
        dist.barrier(group=pg)
        self.validate()

    def validate(self) -> None:
        """Host-side check of the peer pointer table and the flag pad before first use: one
        non-null, distinct base pointer per rank and a flag region that starts out zero."""
        try:
            ptrs = [int(self.hdl.buffer_ptrs[r]) for r in range(self.world)]
        except Exception:          # handle without a host-side pointer list: nothing to check here
            ptrs = None
        if ptrs is not None:
            if any(p == 0 for p in ptrs) or len(set(ptrs)) != self.world:
                raise RuntimeError(f"symmetric workspace: bad peer pointer table {ptrs}")
        if int(self.buf[: self.flag_bytes].view(torch.int32).abs().max().item()) != 0:
            raise RuntimeError("symmetric workspace: flag region is not zero at creation")

    def check_canary(self) -> bool:
        """True while the guard bytes at the end of the workspace are intact."""
        return bool((self.buf[-CANARY_BYTES:] == CANARY_VALUE).all().item())

    def stage(self, x: torch.Tensor, offset: int = 0) -> None:
        """Copy ``x`` (contiguous) into the data region at byte ``offset``."""
        n = x.numel() * x.element_size()
        self.data[offset:offset + n].view(x.dtype).view(x.shape).copy_(x)


class Arena:
    """Symmetric memory that outlives one collective: the gathered activations of the push
    variant of all-gather + GEMM live here, at the same offset on every rank, so that a peer can
    store its rows straight into them. First-fit free list; every rank performs the same sequence
    of ``alloc`` / ``free`` calls (they come from the same recorded schedule), which keeps the
    offsets identical without any exchange."""

    ALIGN = 1 << 20

    def __init__(self, pg, nbytes: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.nbytes = int(nbytes)
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=torch.device("cuda", torch.cuda.current_device()))
        self.hdl = symm_mem.rendezvous(self.buf, group=pg)
        self.ptrs_dev = int(self.hdl.buffer_ptrs_dev)
        self.mc_ptr = 0
        if os.environ.get("NABLA_B200_NVLS", "1") != "0":
            try:
                self.mc_ptr = int(self.hdl.multicast_ptr)
            except Exception:
                self.mc_ptr = 0
        self.free_list: list[list[int]] = [[0, self.nbytes]]      # [offset, size], sorted by offset
        self.live: dict[int, int] = {}
        torch.cuda.synchronize()
        dist.barrier(group=pg)

    def alloc(self, nbytes: int) -> int | None:
        need = (int(nbytes) + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        for i, (off, size) in enumerate(self.free_list):
            if size >= need:
                if size == need:
                    self.free_list.pop(i)
                else:
                    self.free_list[i] = [off + need, size - need]
                self.live[off] = need
                return off
        return None

    def free(self, off: int) -> None:
        size = self.live.pop(off)
        fl = self.free_list
        i = 0
        while i < len(fl) and fl[i][0] < off:
            i += 1
        fl.insert(i, [off, size])
        if i + 1 < len(fl) and fl[i][0] + fl[i][1] == fl[i + 1][0]:
            fl[i][1] += fl[i + 1][1]
            fl.pop(i + 1)
        if i > 0 and fl[i - 1][0] + fl[i - 1][1] == fl[i][0]:
            fl[i - 1][1] += fl[i][1]
            fl.pop(i)


ARENA_BYTES = int(float(os.environ.get("NABLA_B200_SYMM_ARENA_GB", "20")) * (1 << 30))


def arena(mesh, axes) -> Arena | None:
    """The symmetric arena of the device group (created on first use; ``None`` when disabled with
    ``NABLA_B200_SYMM_ARENA_GB=0`` or when the allocation fails)."""
    ws = workspace(mesh, axes)
    if not hasattr(ws, "arena"):
        ws.arena = None
        if ARENA_BYTES > 0:
            try:
                ws.arena = Arena(ws.pg, ARENA_BYTES)
            except Exception:      # not enough memory, or symmetric allocation unsupported
                ws.arena = None
    return ws.arena


_local_only = False


def set_local_only(flag: bool) -> None:
    """Measurement switch: while on, every collective of this module and of ``parallel.backend``
    becomes its communication-free local counterpart with the same shapes (all-reduce = identity,
    all-gather = the own shard repeated, reduce-scatter = the own chunk of the local partial sum,
    fused GEMM + collective = the plain GEMM). A step recorded in this mode does the same math on
    the same tile shapes and moves no byte between GPUs, so ``step time - local-only step time`` is
    the communication a step fails to hide. The numbers it computes are meaningless."""
    global _local_only
    _local_only = bool(flag)


def local_only() -> bool:
    return _local_only


def is_ready() -> bool:
    global _enabled
    if _enabled is None:
        _enabled = False
        if (os.environ.get("NABLA_B200_COMM", "native") != "nccl" and dist.is_available() and dist.is_initialized()
                and torch.cuda.is_available() and dist.get_backend() != "gloo"):
            try:
                from ..native import available

                _enabled = available("libnb_comm.so")
                if _enabled:
                    _L()
            except Exception:
                _enabled = False
    return _enabled


def disable() -> None:
    global _enabled
    _enabled = False


def release_all() -> None:
    """Drop every symmetric workspace and arena of this process (end of a run, all kernels done)."""
    import gc

    for ws in set(_workspaces.values()):
        ws.arena = None
    _workspaces.clear()
    _permute_ws.clear()
    _side_streams.clear()
    gc.collect()


def workspace(mesh, axes) -> Workspace:
    key = (id(mesh), tuple(axes))
    ws = _workspaces.get(key)
    if ws is None:
        pg, ranks = mesh.process_group(tuple(axes))
        # one workspace per set of ranks: ('tp',) and ('dp', 'tp') of a dp=1 mesh share theirs
        ws = _workspaces.get(tuple(ranks))
        if ws is None:
            ws = Workspace(pg, ranks, DEFAULT_BYTES)
            _workspaces[tuple(ranks)] = ws
        _workspaces[key] = ws
    return ws


def supports(buf: torch.Tensor) -> bool:
    return (buf.is_cuda and buf.dtype in (torch.bfloat16, torch.float32)
            and buf.numel() * buf.element_size() + 8192 <= DEFAULT_BYTES - 65536)


def _status():
    from ..native import status_word

    return status_word(torch.device("cuda", torch.cuda.current_device()))


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _blocks_for(nbytes: int) -> int:
    """Grid of the standalone collectives: sized to the bytes NVLink needs in flight (about 2 MB per
    direction at 770 GB/s and a few microseconds of latency; one block keeps 32 KB in flight), not to
    the SM count, and small for latency-bound messages."""
    if nbytes <= 256 * 1024:
        return 8
    if nbytes <= 8 * 1024 * 1024:
        return 32
    return 64 if nbytes <= 64 * 1024 * 1024 else 128


def all_reduce(buf: torch.Tensor, mesh, axes, op: str = "sum", algo: str | None = None) -> torch.Tensor:
    """Sum (or max/min/prod) over the device group of ``axes`` with peer-memory kernels."""
    global launch_count
    if _local_only:
        return buf
    ws = workspace(mesh, axes)
    x = buf.contiguous()
    n = x.numel()
    vec = 16 // x.element_size()
    unit = vec * ws.world
    n_pad = (n + unit - 1) // unit * unit
    flat = x.view(-1)
    region = ws.data[: n_pad * x.element_size()].view(x.dtype)
    region[:n].copy_(flat)
    if n_pad != n:
        region[n:].zero_()
    out = torch.empty(n_pad, dtype=x.dtype, device=x.device)
    nbytes = n_pad * x.element_size()
    opi = {"sum": 0, "max": 1, "min": 2, "prod": 3}[op]
    if algo is None:
        algo = os.environ.get("NABLA_B200_AR_ALGO", "auto")
    if algo == "auto":
        if nbytes <= 512 * 1024 or opi != 0:
            algo = "oneshot"
        else:
            algo = "multimem" if ws.mc_ptr else "twoshot"
    if algo == "multimem" and _deterministic():
        algo = "twoshot"          # peer loads in rank order instead of a sum inside the switch
    if algo == "multimem" and (not ws.mc_ptr or opi != 0):
        algo = "twoshot" if opi == 0 else "oneshot"
    ai = {"oneshot": 0, "twoshot": 1, "multimem": 2}[algo]
    blocks = _blocks_for(nbytes)
    rc = _L().nb_comm_allreduce(ws.ptrs_dev, ws.mc_ptr, ws.rank, ws.world, ws.ctr.data_ptr(), 0, out.data_ptr(), n_pad,
                                1 if x.dtype == torch.bfloat16 else 0, ai, opi, blocks, _status().data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"nb_comm_allreduce failed with code {rc}")
    launch_count += 1
    return out[:n].view(x.shape)


def _deterministic() -> bool:
    from .. import config

    return config.is_deterministic()


_gemm_fn = None
FUSED_COMM_CTAS = int(os.environ.get("NABLA_B200_FUSED_COMM_CTAS", "20"))
AG_COMM_CTAS = int(os.environ.get("NABLA_B200_AG_COMM_CTAS", "12"))
PUSH_COMM_CTAS = int(os.environ.get("NABLA_B200_PUSH_COMM_CTAS", "8"))
MODE_AR, MODE_RS, MODE_AG = 1, 2, 3
_EPI = {"none": 0, "bias": 1, "relu": 2, "gelu": 3}


def _fused_fn():
    global _gemm_fn
    if _gemm_fn is None:
        from ..native import load

        lib = load("libnb_gemm.so")
        fn = lib.nb_gemm_fused_bf16
        fn.restype = c_int
        fn.argtypes = ([c_int] + [c_vp] * 9 + [c_ll, c_int, c_int, c_int, c_int, c_int, c_ll, c_ll] + [c_int] * 9 +
                       [c_vp, c_int, c_vp, c_vp, c_vp, c_ll, c_vp, c_vp])
        lib.nb_gemm_fused_grid.restype = c_int
        _gemm_fn = (fn, lib.nb_gemm_fused_grid)
    return _gemm_fn


def _fused_shapes_ok(m: int, n: int, k: int, nbytes_ws: int) -> bool:
    if n % 8 or k % 8 or m <= 0 or n <= 0 or k <= 0:
        return False
    return nbytes_ws + 4096 <= (DEFAULT_BYTES - 65536) // 2       # the data region is used in two halves


def gemm_all_reduce_supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    """Shapes the fused kernel takes: 2-D bf16 operands, N and K multiples of 8, at most 8192
    output tiles of 128 x 256, output fitting the workspace."""
    if not (a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and b.dim() == 2 and a.dim() >= 2):
        return False
    m, k, n = a.numel() // max(a.shape[-1], 1), a.shape[-1], b.shape[1]
    if m == 0 or ((m + 127) // 128) * ((n + 255) // 256) > 8192:
        return False
    return _fused_shapes_ok(m, n, k, m * n * 2)


def chunked_supported(m_total: int, chunk_rows: int, world: int) -> bool:
    """Row layout the reduce-scatter / all-gather kernels take: whole 128-row tiles per chunk."""
    return chunk_rows > 0 and chunk_rows % 128 == 0 and m_total % (world * chunk_rows) == 0 and m_total // 128 <= 2048


_side_streams: dict = {}


def _side_stream(device) -> "torch.cuda.Stream":
    st = _side_streams.get(device)
    if st is None:
        st = torch.cuda.Stream(device=device)
        _side_streams[device] = st
    return st


def _fused_state(ws, device):
    if not hasattr(ws, "ticket"):
        ws.ticket = torch.zeros(4, dtype=torch.int32, device=device)
    return ws


def _launch_fused(mode, ws, a, b, out, bias, aux_out, a_full, M, N, K, lda, ldb, a_mn, b_mn, epi, aux, gelu_tanh,
                  chunk_rows, n_comm, arena_ptrs: int = 0, a_off: int = 0, arena_mc: int = 0):
    """Returns the byte offset (inside the workspace) of the region the call used."""
    global launch_count
    fn, grid_fn = _fused_fn()
    lib = _L()
    grid = grid_fn()
    n_comm = max(1, min(n_comm, grid // 2))
    data_off = ws.flag_bytes
    if mode != MODE_AG:
        # calls that write into the peers' workspaces alternate between two halves: the local
        # fold of call n (which runs after the kernel's closing barrier) may still be reading its
        # half when a faster peer already pushes tiles of call n + 1
        half = ((ws.nbytes - ws.flag_bytes) // 2) & ~1023
        if M * N * 2 > half:
            raise RuntimeError(f"fused GEMM+collective output ({M}x{N}) does not fit half of the workspace")
        ws.parity = 1 - getattr(ws, "parity", 1)
        data_off += ws.parity * half
    p = lambda t: c_vp(0 if t is None else t.data_ptr())
    # deterministic replay: reduce jobs in a fixed order (no ticket counter), partial tiles added with
    # peer loads in rank order (no multicast pointer)
    det = _deterministic()
    rc = fn(mode, p(a), p(b), p(out), p(bias), p(aux_out), p(a_full), ws.buf.data_ptr(), ws.ptrs_dev,
            0 if det else ws.mc_ptr,
            data_off, lib.nb_comm_tile_flag_offset(), lib.nb_comm_done_offset(), M, N, K, lda, ldb, a_mn, b_mn,
            1 if (bias is not None and bias.dtype == torch.float32) else 0, epi, aux, int(gelu_tanh), ws.rank, ws.world,
            chunk_rows, ws.ctr.data_ptr(), n_comm, 0 if det else ws.ticket.data_ptr(), _status().data_ptr(), arena_ptrs,
            a_off, 0 if det else arena_mc, _stream())
    if rc != 0:
        raise RuntimeError(f"nb_gemm_fused_bf16(mode={mode}) failed with code {rc} for M={M} N={N} K={K}")
    launch_count += 1
    return data_off


def _operands(a: torch.Tensor, b: torch.Tensor):
    from ..native.gemm import _prep

    a2 = a.reshape(-1, a.shape[-1])
    a3, akind, lda, _ = _prep(a2.unsqueeze(0))
    b3, bkind, ldb, _ = _prep(b.unsqueeze(0))
    return a3, b3, lda, ldb, (0 if akind == "row" else 1), (1 if bkind == "row" else 0)


def gemm_all_reduce(a: torch.Tensor, b: torch.Tensor, mesh, axes) -> torch.Tensor:
    """``sum over the group of (a_r @ b_r)`` in ONE kernel: the tcgen05 GEMM writes each output
    tile into the symmetric workspace and counts it on the tile's owner; reduction CTAs of the
    same launch sum finished tiles through the switch (``multimem.ld_reduce`` + ``multimem.st``)
    or over plain peer loads/stores while later tiles are still being multiplied.

    Returns a VIEW of the workspace (M x N bf16): consume or copy it before the next collective
    on this group."""
    if _local_only:
        from ..native.gemm import gemm_bf16

        return gemm_bf16(a.reshape(-1, a.shape[-1]), b)
    ws = _fused_state(workspace(mesh, axes), a.device)
    a3, b3, lda, ldb, a_mn, b_mn = _operands(a, b)
    M, K, N = a3.shape[1], a3.shape[2], b.shape[1]
    off = _launch_fused(MODE_AR, ws, a3, b3, None, None, None, None, M, N, K, lda, ldb, a_mn, b_mn, 0, 0, False, 0,
                        FUSED_COMM_CTAS)
    return ws.buf[off: off + M * N * 2].view(torch.bfloat16).view(M, N)


def gemm_reduce_scatter(a: torch.Tensor, b: torch.Tensor, mesh, axes, chunk_rows: int,
                        bias: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
    """Rows of ``sum_r a_r @ b_r`` (+ ``bias`` + ``residual``) that belong to this rank (row
    chunks of ``chunk_rows`` dealt round-robin to the ranks). The GEMM's epilogue stores every
    output tile straight into the memory of the rank that owns its rows (peer stores over NVLink,
    overlapped with the next tile's MMAs; no SM is set aside for communication); after the
    launch's closing barrier a local pass folds the ``world`` partial row blocks, the bias and
    the residual into the returned (M / world, N) tensor."""
    ws = _fused_state(workspace(mesh, axes), a.device)
    if _local_only:
        from ..native.gemm import gemm_bf16

        y = gemm_bf16(a.reshape(-1, a.shape[-1]), b)
        M, N = y.shape
        own = y.view(M // (ws.world * chunk_rows), ws.world, chunk_rows, N)[:, ws.rank]     # strided view, no copy
        # one pass like the real kernel's fold: own chunk (+ residual) -> contiguous, bias added in place
        out = torch.add(own, residual.reshape(own.shape)) if residual is not None else own.contiguous()
        if bias is not None:
            out.add_(bias.reshape(-1).to(out.dtype))
        return out.reshape(M // ws.world, N)
    a3, b3, lda, ldb, a_mn, b_mn = _operands(a, b)
    M, K, N = a3.shape[1], a3.shape[2], b.shape[1]
    out = torch.empty((M // ws.world, N), dtype=torch.bfloat16, device=a.device)
    if bias is not None:
        bias = bias.reshape(-1).to(torch.bfloat16).contiguous()
    if residual is not None:
        residual = residual.reshape(M // ws.world, N).contiguous()
    _launch_fused(MODE_RS, ws, a3, b3, out, bias, residual, None, M, N, K, lda, ldb, a_mn, b_mn, 0, 0, False,
                  chunk_rows, 1)
    return out


def all_gather_gemm(a_shard: torch.Tensor, b: torch.Tensor, mesh, axes, chunk_rows: int, bias: torch.Tensor | None = None,
                    epilogue: str = "none", gelu_tanh: bool = False, store_preact: bool = False,
                    comm_ctas: int | None = None, arena_off: int | None = None, dact: tuple | None = None):
    """``epilogue(gather(a) @ b + bias)`` in one kernel. ``a_shard`` is this rank's rows
    (M / world, K). The tensor-core CTAs start on the own rows (read in place) while copy CTAs of
    the same launch move the other rows over NVLink; each later tile waits only for its own
    128-row block.

    Two copy directions. With ``arena_off`` (an offset in the group's symmetric :class:`Arena`,
    the same on every rank) the gathered matrix lives in the arena and every rank PUSHES its rows
    into all peers' copies with posted bulk stores: no round trip to wait for, a handful of copy
    CTAs keep the link busy, and nothing has to be staged. Without it the rows are staged in the
    workspace and PULLED by the consumer (bulk loads through shared memory).

    ``dact=(z, activation)`` multiplies the product by ``activation'(z)`` in the epilogue (the
    backward of a fused linear + activation; ``z`` is (M, N)).

    Returns ``(a_full, out)`` or ``(a_full, out, preact)``; ``a_full`` (M, K) is the all-gather's
    own result, kept for the backward pass."""
    from ..native.gemm import _prep

    ws = _fused_state(workspace(mesh, axes), a_shard.device)
    x = a_shard.reshape(-1, a_shard.shape[-1]).contiguous()
    Ml, K = x.shape
    M, N = Ml * ws.world, b.shape[1]
    if _local_only:
        from ..native.gemm import gemm_bf16

        if arena_off is not None:
            a_full = ws.arena.buf[arena_off: arena_off + M * K * 2].view(torch.bfloat16).view(M, K)
        else:
            a_full = torch.empty((M, K), dtype=torch.bfloat16, device=x.device)
        # the gathered matrix is left as it is (stale or uninitialised rows): the GEMM reads the same bytes
        # from the same place as in the real step, and no copy that the real step does not make is added
        if bias is not None and epilogue == "none":
            epilogue = "bias"
        if dact is not None:
            z, act = dact
            o = gemm_bf16(a_full, b, aux="drelu" if act == "relu" else "dgelu", aux_in=z.reshape(M, N),
                          gelu_tanh=act == "gelu_tanh")
            return a_full, o
        if store_preact:
            o, pre = gemm_bf16(a_full, b, bias=bias, epilogue=epilogue, aux="store_preact", gelu_tanh=gelu_tanh)
            return a_full, o, pre
        return a_full, gemm_bf16(a_full, b, bias=bias, epilogue=epilogue, gelu_tanh=gelu_tanh)
    b3, bkind, ldb, _ = _prep(b.unsqueeze(0))
    push = arena_off is not None
    if push:
        ar = ws.arena
        a_full = ar.buf[arena_off: arena_off + M * K * 2].view(torch.bfloat16).view(M, K)
    else:
        ws.data[: Ml * K * 2].view(torch.bfloat16).view(Ml, K).copy_(x)        # stage where peers can read it
        a_full = torch.empty((M, K), dtype=torch.bfloat16, device=x.device)
    out = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    pre = torch.empty((M, N), dtype=torch.bfloat16, device=x.device) if store_preact else None
    if bias is not None:
        bias = bias.reshape(-1).contiguous()
        if epilogue == "none":
            epilogue = "bias"
    # With a multicast binding of the arena one multimem.st per 16 bytes reaches the gathered matrix of
    # every rank (this one included) through the switch: the rows leave the GPU once, not world - 1 times.
    # Measured: with two ranks the multicast push wins (0.48 ms against 0.63 ms for 32768 x 4096 x 2048);
    # with four the receiving side is the limit either way and plain peer stores from 16 copy CTAs are
    # faster (0.43 ms against 0.57 ms for 65536 x 1536 x 2048), so multicast is the default for pairs only.
    mm = os.environ.get("NABLA_B200_AG_MULTIMEM", "auto")
    arena_mc = ws.arena.mc_ptr if (push and (mm == "1" or (mm == "auto" and ws.world == 2))) else 0
    if _deterministic():
        arena_mc = 0
    cs = chunk_rows
    cur = torch.cuda.current_stream()
    side = cur if _deterministic() else _side_stream(x.device)
    if not arena_mc:
        # this rank's own rows of the gathered matrix (the kernel moves only the peers' rows): a plain
        # copy on a side stream, issued first so that it runs under the fused kernel (which reads the
        # own rows from ``x``, not from here); the streams join again right after the launch
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            a_full.view(M // (ws.world * cs), ws.world, cs, K)[:, ws.rank].copy_(x.view(-1, cs, K))
    # copy CTAs: an SM moves about 32 GB/s (pull) to 38 GB/s (push); take as many as it needs to move
    # its share within the GEMM's own time, up to what saturates the link
    if comm_ctas is None:
        gemm_s = 2.0 * M * N * K / 1.5e15          # the GEMM's own time on CTA pairs
        out_bytes = Ml * K * 2 if arena_mc else (M - Ml) * K * 2
        need = out_bytes / max(gemm_s, 1e-6) / (38e9 if push else 32e9)
        # measured: below 8 copy CTAs a multicast push does not keep up with the GEMM (0.57 ms with 5,
        # 0.48 ms with 8 or more for 32768 x 4096 x 2048 on two GPUs, GEMM alone 0.44 ms)
        comm_ctas = int(min(20, max(8 if arena_mc else 4, need + 1.5)))
    n_comm = comm_ctas
    aux_code, aux_t = (1 if store_preact else 0), pre
    if dact is not None:
        z, act = dact
        aux_t = z.reshape(M, N).contiguous()
        aux_code = 2 if act == "relu" else 3
        gelu_tanh = act == "gelu_tanh"
    _launch_fused(MODE_AG, ws, x, b3, out, bias, aux_t, a_full, M, N, K, K, ldb, 0, 1 if bkind == "row" else 0,
                  _EPI[epilogue], aux_code, gelu_tanh, chunk_rows, n_comm,
                  ws.arena.ptrs_dev if push else 0, arena_off or 0, arena_mc)
    if not arena_mc:
        cur.wait_stream(side)
    return (a_full, out, pre) if store_preact else (a_full, out)


def adamw_reduce(p: torch.Tensor, m: torch.Tensor, v: torch.Tensor, grad_off: int, mesh, axes, *, lr: float, b1: float,
                 b2: float, eps: float, wd: float, step: int | None = None, hyper: torch.Tensor | None = None,
                 grad_scale: float = 1.0) -> None:
    """Data-parallel AdamW step of one parameter in ONE kernel: the ranks' bf16 gradients sit at
    ``grad_off`` of the group's symmetric :class:`Arena`; the kernel sums them over NVLink while it
    reads them (``multimem.ld_reduce`` or one load per peer), applies scale + AdamW to ``p`` (bf16),
    ``m``, ``v`` (fp32) in place, and brackets itself with the two barriers that keep the gradients
    valid. Replaces all-reduce + cast + AdamW (reference: nabla/nn/optim/functional.py:116-162 after
    the partial-sum all-reduce of nabla/core/autograd/backward.py:72-80)."""
    global launch_count
    ws = _fused_state(workspace(mesh, axes), p.device)
    ar = ws.arena
    n = p.numel()
    if _local_only:
        from ..native import kernels

        g = ar.buf[grad_off: grad_off + n * 2].view(torch.bfloat16).view(p.shape)
        kernels.adamw(p, g, m, v, lr=lr, b1=b1, b2=b2, eps=eps, wd=wd, step=step or 1, inplace=True)
        return
    bc1 = 1.0 - b1 ** step if step is not None else 1.0
    bc2 = 1.0 - b2 ** step if step is not None else 1.0
    blocks = int(max(1, min(256, (n // 8 + 255) // 256)))
    rc = _L().nb_comm_adamw_reduce(ws.ptrs_dev, ws.rank, ws.world, ws.ctr.data_ptr(), ar.ptrs_dev, 0 if _deterministic() else ar.mc_ptr, grad_off,
                                   p.data_ptr(), m.data_ptr(), v.data_ptr(), n, float(lr), float(b1), float(b2),
                                   float(eps), float(wd), float(bc1), float(bc2), float(grad_scale),
                                   c_vp(0 if hyper is None else hyper.data_ptr()), blocks, _status().data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"nb_comm_adamw_reduce failed with code {rc}")
    launch_count += 1


def _gather_call(x: torch.Tensor, mesh, axes, mode: int, chunk_elems: int, out_elems: int, root: int = 0) -> torch.Tensor:
    global launch_count
    ws = workspace(mesh, axes)
    flat = x.contiguous().view(-1)
    if _local_only:
        if mode == 0:                                     # all-gather: the own shard repeated
            return flat.repeat(ws.world)
        if mode == 1:                                     # reduce-scatter: own chunk of the local partial sum
            return flat[ws.rank * chunk_elems:(ws.rank + 1) * chunk_elems].clone()
        return flat.clone()
    ws.data[: flat.numel() * x.element_size()].view(x.dtype).copy_(flat)
    out = torch.empty(out_elems, dtype=x.dtype, device=x.device)
    nbytes = out_elems * x.element_size()
    blocks = _blocks_for(nbytes)
    rc = _L().nb_comm_gather(ws.ptrs_dev, ws.rank, ws.world, ws.ctr.data_ptr(), 0, out.data_ptr(), chunk_elems,
                             1 if x.dtype == torch.bfloat16 else 0, mode, root, blocks, _status().data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"nb_comm_gather failed with code {rc}")
    launch_count += 1
    return out


PERMUTE_SLOT_BYTES = int(os.environ.get("NABLA_B200_PERMUTE_SLOT_MB", "32")) * 1024 * 1024
_permute_ws: dict = {}


def _permute_workspace(mesh) -> Workspace:
    """The whole mesh's workspace for point-to-point shifts: the flag pad and two inbox slots. No other
    collective uses it, which is what lets ``permute_kernel`` get by with one barrier per call."""
    axes = tuple(mesh.axis_names)
    pg, ranks = mesh.process_group(axes)
    ws = _permute_ws.get(tuple(ranks))
    if ws is None:
        ws = Workspace(pg, ranks, _L().nb_comm_flag_bytes() + 2 * PERMUTE_SLOT_BYTES + CANARY_BYTES + 4096)
        _permute_ws[tuple(ranks)] = ws
    return ws


def permute_supported(buf: torch.Tensor, mesh, perm) -> bool:
    """One launch of the peer-memory shift handles a (partial) permutation of the mesh's ranks whose
    payload is a whole number of 16-byte vectors and fits an inbox slot."""
    srcs = [s for s, _ in perm]
    dsts = [d for _, d in perm]
    nbytes = buf.numel() * buf.element_size()
    return (buf.is_cuda and len(set(srcs)) == len(srcs) and len(set(dsts)) == len(dsts)
            and nbytes % 16 == 0 and 0 < nbytes <= PERMUTE_SLOT_BYTES)


def permute(buf: torch.Tensor, mesh, perm) -> torch.Tensor:
    """Point-to-point shift over the whole mesh with one peer-memory kernel (`permute_kernel`):
    rank ``s`` stores its buffer into rank ``d``'s inbox for every pair ``(s, d)``; ranks nobody
    sends to get zeros. Every rank of the mesh makes the call, whether it sends, receives or neither
    (reference: nabla/ops/communication/p_permute.py:85-119, a device-to-device copy per pair)."""
    global launch_count
    ws = _permute_workspace(mesh)
    ranks = ws.ranks
    me = mesh.rank
    dst = next((d for s, d in perm if s == me), None)
    src = next((s for s, d in perm if d == me), None)
    x = buf.contiguous()
    own = dst == me                                 # a fixed point of the permutation: nothing crosses a link,
    if own:                                         # but the rank still meets the others at the barrier
        dst = src = None
    out = torch.empty_like(x)
    nbytes = x.numel() * x.element_size()
    rc = _L().nb_comm_permute(ws.ptrs_dev, ws.rank, ws.world, ws.ctr.data_ptr(), PERMUTE_SLOT_BYTES, x.data_ptr(),
                              out.data_ptr(), nbytes, -1 if dst is None else ranks.index(dst),
                              -1 if src is None else ranks.index(src), 8 if nbytes <= (1 << 20) else 32,
                              _status().data_ptr(), _stream())
    if rc != 0:
        raise RuntimeError(f"nb_comm_permute failed with code {rc}")
    launch_count += 1
    return x.clone() if own else out


def all_gather_dim0(x: torch.Tensor, mesh, axes) -> torch.Tensor:
    """Concatenate equal-size shards along dim 0 (numel a multiple of 16 bytes)."""
    ws = workspace(mesh, axes)
    out = _gather_call(x, mesh, axes, 0, x.numel(), x.numel() * ws.world)
    return out.view((x.shape[0] * ws.world,) + tuple(x.shape[1:]))


def reduce_scatter_dim0(x: torch.Tensor, mesh, axes) -> torch.Tensor:
    ws = workspace(mesh, axes)
    chunk = x.numel() // ws.world
    out = _gather_call(x, mesh, axes, 1, chunk, chunk)
    return out.view((x.shape[0] // ws.world,) + tuple(x.shape[1:]))


def all_to_all_dim0(x: torch.Tensor, mesh, axes) -> torch.Tensor:
    ws = workspace(mesh, axes)
    chunk = x.numel() // ws.world
    return _gather_call(x, mesh, axes, 2, chunk, x.numel()).view(x.shape)


def broadcast(x: torch.Tensor, mesh, axes, root: int = 0) -> torch.Tensor:
    return _gather_call(x, mesh, axes, 3, x.numel(), x.numel(), root).view(x.shape)


def wait_flag_timeout_probe(limit_ms: float = 50.0) -> int:
    """Launch a bounded wait on a flag nobody sets; returns the status code the kernel reported
    (NB_ERR_TIMEOUT_PEER = 4). The CUDA context stays usable: this is how lost-peer detection is
    tested without faulting or hanging a GPU."""
    dev = torch.device("cuda", torch.cuda.current_device())
    flag = torch.zeros(4, dtype=torch.int32, device=dev)
    st = torch.zeros(4, dtype=torch.int32, device=dev)
    rc = _L().nb_comm_wait_flag(flag.data_ptr(), 1, st.data_ptr(), int(limit_ms * 1e6), _stream())
    if rc != 0:
        raise RuntimeError("wait_flag launch failed")
    torch.cuda.synchronize()
    return int(st[0].item())
