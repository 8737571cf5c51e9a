"""Distributed API with the reference's semantics (Tyr/Distributed.lean, cc/src/tyr_distributed.cpp).

* ``init_process_group`` validates backend / port / rank / world size BEFORE any rendezvous.
* Collectives have value semantics: they work on a private clone and return a fresh tensor; the
  input is never modified (Distributed.lean:43-78).
* Async variants return a ``WorkHandle``; the handle is removed from the pending table before it
  is waited on, so it is released exactly once even if waiting raises; ``destroy_process_group``
  drains everything still pending, resets the state and re-raises the first error.
* ``reduce_scatter`` splits dim 0 of the input, ``all_gather`` concatenates on dim 0.

Transport is torch's c10d (NCCL on GPU, Gloo on CPU); id/lifecycle bookkeeping is native
(csrc/host/pg_registry.cpp).  The hot training path does not use these calls: see
:mod:`tyr_b200.parallel.dp` for the fused NVLink kernels.
"""
from __future__ import annotations

import contextlib
import ctypes
import enum
import os
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as tdist

from .._native import host, register_host_signatures
from .sampler import DistributedSampler, DistributedSamplerConfig  # noqa: F401


# Transport callbacks handed to the native lifecycle (csrc/host/pg_registry.cpp): it decides the order of operations,
# these only talk to c10d.  Each returns 0, or records its error natively and returns 1; the Python exception object is
# kept aside so that the caller can chain it.
_RENDEZVOUS_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)
_WAIT_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p, ctypes.c_uint64)
_SHUTDOWN_FN = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_void_p)


@register_host_signatures
def _sigs(lib):
    L, U = ctypes.c_longlong, ctypes.c_uint64
    lib.tyr_pg_validate_init.argtypes = [ctypes.c_char_p, ctypes.c_char_p, L, L, L]
    lib.tyr_pg_mark_initialized.argtypes = [L, L]
    lib.tyr_pg_register_work.restype = U
    lib.tyr_pg_take_work.argtypes = [U]
    lib.tyr_pg_has_work.argtypes = [U]
    lib.tyr_pg_pending_count.restype = L
    lib.tyr_pg_pending_ids.argtypes = [ctypes.POINTER(U), L]
    lib.tyr_pg_pending_ids.restype = L
    lib.tyr_pg_record_error.argtypes = [ctypes.c_char_p]
    lib.tyr_pg_record_error.restype = None
    lib.tyr_pg_first_error.argtypes = [ctypes.c_char_p, L]
    lib.tyr_pg_first_error.restype = L
    lib.tyr_pg_init.argtypes = [ctypes.c_char_p, ctypes.c_char_p, L, L, L, _RENDEZVOUS_FN, ctypes.c_void_p]
    lib.tyr_pg_wait.argtypes = [U, _WAIT_FN, ctypes.c_void_p]
    lib.tyr_pg_destroy.argtypes = [_WAIT_FN, _SHUTDOWN_FN, ctypes.c_void_p]


_last_exc: List[Optional[BaseException]] = [None]


def _native_error() -> str:
    buf = ctypes.create_string_buffer(2048)
    host().tyr_pg_first_error(buf, 2048)
    return buf.value.decode(errors="replace")


def _guard(fn):
    """Wrap a transport action as a callback body: exceptions become a recorded native error + return code 1."""
    def run(*args):
        try:
            fn(*args)
            return 0
        except BaseException as e:  # noqa: BLE001 - crossing a C frame: never propagate
            if _last_exc[0] is None:
                _last_exc[0] = e
            host().tyr_pg_record_error(f"{type(e).__name__}: {e}".encode(errors="replace")[:2000])
            return 1
    return run


class ReduceOp(enum.Enum):
    sum = "sum"
    avg = "avg"
    product = "product"
    min = "min"
    max = "max"


class DistributedError(RuntimeError):
    pass


class _TorchBackend:
    """Thin adapter over torch.distributed so tests can substitute a fake."""

    def __init__(self, group=None):
        self.group = group

    def rank(self):
        return tdist.get_rank(self.group)

    def size(self):
        return tdist.get_world_size(self.group)

    def _op(self, op: ReduceOp):
        return {ReduceOp.sum: tdist.ReduceOp.SUM, ReduceOp.avg: tdist.ReduceOp.SUM,
                ReduceOp.product: tdist.ReduceOp.PRODUCT, ReduceOp.min: tdist.ReduceOp.MIN,
                ReduceOp.max: tdist.ReduceOp.MAX}[op]

    def all_reduce(self, t, op, async_op):
        return tdist.all_reduce(t, self._op(op), group=self.group, async_op=async_op)

    def broadcast(self, t, root, async_op):
        return tdist.broadcast(t, root, group=self.group, async_op=async_op)

    def reduce_scatter_tensor(self, out, inp, op, async_op):
        if inp.is_cuda:
            return tdist.reduce_scatter_tensor(out, inp, self._op(op), group=self.group, async_op=async_op)
        # Gloo has no reduce_scatter: all_reduce + slice (test transport only)
        tmp = inp.clone()
        tdist.all_reduce(tmp, self._op(op), group=self.group)
        n = out.shape[0]
        out.copy_(tmp[self.rank() * n:(self.rank() + 1) * n])
        return None

    def reduce_scatter_list(self, out, inputs, op, async_op):
        if out.is_cuda:
            return tdist.reduce_scatter(out, list(inputs), self._op(op), group=self.group, async_op=async_op)
        tmp = [t.clone() for t in inputs]
        for t in tmp:
            tdist.all_reduce(t, self._op(op), group=self.group)
        out.copy_(tmp[self.rank()])
        return None

    def all_gather_into_tensor(self, out, inp, async_op):
        if inp.is_cuda:
            return tdist.all_gather_into_tensor(out, inp, group=self.group, async_op=async_op)
        parts = [torch.empty_like(inp) for _ in range(self.size())]
        tdist.all_gather(parts, inp, group=self.group)
        out.copy_(torch.cat(parts, dim=0))
        return None

    def all_gather_list(self, outs, inp, async_op):
        return tdist.all_gather(outs, inp, group=self.group, async_op=async_op)

    def barrier(self):
        tdist.barrier(group=self.group)

    def shutdown(self):
        if tdist.is_initialized():
            tdist.destroy_process_group()


_backend = None
_works: Dict[int, object] = {}
_owns_torch_pg = False


def _lib():
    return host()


def _require():
    if _backend is None:
        raise DistributedError("process group is not initialised")
    return _backend


_INIT_ERRORS = {1: "unsupported backend (expected 'nccl' or 'gloo')", 2: "port must be in 1..65535",
                3: "world size must be positive", 4: "rank must satisfy 0 <= rank < world size",
                5: "master address is empty", 6: "process group is already initialised"}


def validate_init(backend: str, master_addr: str, master_port: int, rank: int, world_size: int) -> None:
    rc = _lib().tyr_pg_validate_init(backend.encode(), master_addr.encode(), master_port, rank, world_size)
    if rc != 0:
        raise ValueError(f"initProcessGroup: {_INIT_ERRORS.get(rc, 'invalid arguments')}")


def set_cuda_device(local_rank: int) -> None:
    if not torch.cuda.is_available():
        raise DistributedError("setCudaDevice: CUDA is not available")
    if not 0 <= local_rank < torch.cuda.device_count():
        raise DistributedError(f"setCudaDevice: ordinal {local_rank} out of range")
    torch.cuda.set_device(local_rank)


def init_process_group(backend: str, master_addr: str = "127.0.0.1", master_port: int = 29500, rank: int = 0,
                       world_size: int = 1, timeout_s: float = 600.0, _inject=None) -> None:
    """Validates first, then performs the TCPStore rendezvous and builds the communicator."""
    global _backend, _owns_torch_pg
    made = {}

    def rendezvous(_ctx):
        if _inject is not None:
            made["backend"] = _inject
            return
        import datetime
        if not tdist.is_initialized():
            tdist.init_process_group(backend, init_method=f"tcp://{master_addr}:{master_port}", rank=rank,
                                     world_size=world_size, timeout=datetime.timedelta(seconds=timeout_s))
            made["owns"] = True
        made["backend"] = _TorchBackend()

    _last_exc[0] = None
    cb = _RENDEZVOUS_FN(_guard(rendezvous))
    rc = _lib().tyr_pg_init(backend.encode(), master_addr.encode(), master_port, rank, world_size, cb, None)
    if 1 <= rc <= 6:
        raise ValueError(f"initProcessGroup: {_INIT_ERRORS.get(rc, 'invalid arguments')}")
    if rc != 0:
        exc, _last_exc[0] = _last_exc[0], None
        raise DistributedError(f"initProcessGroup: {_native_error()}") from exc
    _backend = made["backend"]
    _owns_torch_pg = bool(made.get("owns", False))


def is_initialized() -> bool:
    return _backend is not None


def registry_state():
    """(initialised, rank, world) as recorded by the native registry that survives Python-side resets; the
    counterpart of the globals in cc/src/tyr_distributed.cpp:49-58."""
    lib = _lib()
    return bool(lib.tyr_pg_is_initialized()), int(lib.tyr_pg_rank()), int(lib.tyr_pg_world())


def get_rank() -> int:
    return _require().rank()


def get_world_size() -> int:
    return _require().size()


def destroy_process_group() -> None:
    """Drain every pending handle, reset, then re-raise the first error seen while draining."""
    global _backend, _owns_torch_pg, _peer
    if _peer is not None:
        # every peer collective ends with a barrier after the last peer read, so the staging heap is idle here
        try:
            torch.cuda.synchronize(_peer.device)
            _peer.close()
        finally:
            _peer = None

    def wait_one(_ctx, hid):
        _wait_transport(int(hid))

    def shutdown(_ctx):
        if _backend is not None and (_owns_torch_pg or not isinstance(_backend, _TorchBackend)):
            _backend.shutdown()

    _last_exc[0] = None
    wcb, scb = _WAIT_FN(_guard(wait_one)), _SHUTDOWN_FN(_guard(shutdown))
    rc = _lib().tyr_pg_destroy(wcb, scb, None)        # drain -> shutdown -> reset, first error kept natively
    _backend = None
    _owns_torch_pg = False
    _works.clear()
    if rc != 0:
        exc, _last_exc[0] = _last_exc[0], None
        raise DistributedError(f"destroyProcessGroup: pending work failed: {_native_error()}") from exc


class WorkHandle:
    """Result of an async collective.  The tensor is only observable through ``wait()``."""

    def __init__(self, hid: int):
        self.id = hid

    def wait(self) -> torch.Tensor:
        out = {}

        def wait_one(_ctx, hid):
            out["v"] = _wait_transport(int(hid))

        _last_exc[0] = None
        rc = _lib().tyr_pg_wait(self.id, _WAIT_FN(_guard(wait_one)), None)     # erase-before-wait happens natively
        if rc == 1:
            raise DistributedError(f"wait: unknown or already consumed work handle {self.id}")
        if rc != 0:
            exc, _last_exc[0] = _last_exc[0], None
            if isinstance(exc, DistributedError):
                raise exc
            raise DistributedError(f"wait: {_native_error()}") from exc
        return out["v"]

    def is_completed(self) -> bool:
        if not _lib().tyr_pg_has_work(self.id):
            return True
        work = _works[self.id][0]
        if work is None:
            return True
        done = work.is_completed()
        if done and hasattr(work, "exception") and callable(work.exception) and work.exception() is not None:
            return True
        return bool(done)


def _wait_transport(hid: int):
    """Wait on the c10d work object behind a handle that the native table has already released."""
    work, result, post = _works.pop(hid)
    if work is not None:
        ok = work.wait()
        if ok is False:
            raise DistributedError("collective was aborted")
    return post(result) if post else result


def _submit(work, result, post=None) -> WorkHandle:
    hid = int(_lib().tyr_pg_register_work())
    _works[hid] = (work, result, post)
    return WorkHandle(hid)


def wait_all(handles: Sequence[WorkHandle]) -> List[torch.Tensor]:
    return [h.wait() for h in handles]


def barrier() -> None:
    _require().barrier()


def _avg_post(op: ReduceOp, world: int):
    if op is not ReduceOp.avg:
        return None

    def post(t):
        return (t / world).to(t.dtype) if t.dtype.is_floating_point else torch.div(t, world, rounding_mode="floor")
    return post


# ---- peer-memory collectives (distributed/peer.py) --------------------------------------------------------------
_peer = None


def enable_peer_collectives(capacity_bytes: int = 256 << 20, device=None):
    """Routes ``all_reduce`` / ``reduce_scatter(_list)`` / ``all_gather(_list)`` of floating-point CUDA tensors (sum and
    avg) through the hand-written peer-memory kernels instead of NCCL.  Collective: every rank calls it, once, after
    ``init_process_group``; needs one process per GPU on one node.  Returns the ``PeerCollectives`` object."""
    global _peer
    b = _require()
    if _peer is None:
        from .peer import PeerCollectives
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        _peer = PeerCollectives(b.rank(), b.size(), dev, capacity_bytes, getattr(b, "group", None))
    return _peer


def disable_peer_collectives() -> None:
    global _peer
    if _peer is not None:
        torch.cuda.synchronize(_peer.device)
        barrier()
        _peer.close()
        _peer = None


def _use_peer(t: torch.Tensor, op: ReduceOp, copies: int = 1) -> bool:
    return _peer is not None and op in (ReduceOp.sum, ReduceOp.avg) and _peer.supports(t, copies)


class _Done:
    """Stands in for a transport work object when the result was produced by stream-ordered kernels."""

    def wait(self):
        return True

    def is_completed(self):
        return True


def all_reduce_async(t: torch.Tensor, op: ReduceOp = ReduceOp.sum) -> WorkHandle:
    b = _require()
    if _use_peer(t, op):
        return _submit(_Done(), _peer.all_reduce(t, op is ReduceOp.avg))
    out = t.detach().clone()
    work = b.all_reduce(out, op, True)
    return _submit(work, out, _avg_post(op, b.size()))


def all_reduce(t: torch.Tensor, op: ReduceOp = ReduceOp.sum) -> torch.Tensor:
    r = all_reduce_async(t, op).wait()
    return r.requires_grad_(t.requires_grad) if t.requires_grad else r


def broadcast(t: torch.Tensor, root: int = 0) -> torch.Tensor:
    b = _require()
    if not 0 <= root < b.size():
        raise ValueError(f"broadcast: root {root} outside the world of {b.size()}")
    out = t.detach().clone()
    b.broadcast(out, root, False)
    return out.requires_grad_(t.requires_grad) if t.requires_grad else out


def reduce_scatter(t: torch.Tensor, op: ReduceOp = ReduceOp.sum) -> torch.Tensor:
    """Splits dim 0 of ``t`` into world chunks; returns this rank's reduced chunk."""
    b = _require()
    W = b.size()
    if t.dim() == 0 or t.shape[0] % W != 0:
        raise ValueError(f"reduceScatter: dim 0 of {list(t.shape)} does not divide by world size {W}")
    if _use_peer(t, op):
        return _peer.reduce_scatter(t, op is ReduceOp.avg)
    inp = t.detach().clone().contiguous()
    out = torch.empty((t.shape[0] // W,) + tuple(t.shape[1:]), dtype=t.dtype, device=t.device)
    b.reduce_scatter_tensor(out, inp, op, False)
    post = _avg_post(op, W)
    return post(out) if post else out


def reduce_scatter_list(ts: Sequence[torch.Tensor], op: ReduceOp = ReduceOp.sum) -> torch.Tensor:
    b = _require()
    W = b.size()
    if len(ts) != W:
        raise ValueError(f"reduceScatterList: expected {W} tensors, got {len(ts)}")
    if any(x.shape != ts[0].shape or x.dtype != ts[0].dtype for x in ts):
        raise ValueError("reduceScatterList: tensors must share shape and dtype")
    if _use_peer(ts[0], op, W):
        return _peer.reduce_scatter_list(ts, op is ReduceOp.avg)
    ins = [x.detach().clone().contiguous() for x in ts]
    out = torch.empty_like(ins[0])
    b.reduce_scatter_list(out, ins, op, False)
    post = _avg_post(op, W)
    return post(out) if post else out


def all_gather(t: torch.Tensor) -> torch.Tensor:
    """Concatenation of every rank's tensor along dim 0."""
    b = _require()
    if _use_peer(t, ReduceOp.sum):
        return _peer.all_gather(t)
    inp = t.detach().clone().contiguous()
    if inp.dim() == 0:
        inp = inp.reshape(1)
    out = torch.empty((inp.shape[0] * b.size(),) + tuple(inp.shape[1:]), dtype=inp.dtype, device=inp.device)
    b.all_gather_into_tensor(out, inp, False)
    return out


def all_gather_list(t: torch.Tensor) -> List[torch.Tensor]:
    b = _require()
    if _use_peer(t, ReduceOp.sum):
        return _peer.all_gather_list(t)
    inp = t.detach().clone().contiguous()
    outs = [torch.empty_like(inp) for _ in range(b.size())]
    b.all_gather_list(outs, inp, False)
    return outs


@contextlib.contextmanager
def with_distributed(backend: str, master_addr: str, master_port: int, rank: int, world_size: int):
    """Bracketed form: always tears down (Distributed.lean:173-183)."""
    init_process_group(backend, master_addr, master_port, rank, world_size)
    try:
        yield
    finally:
        destroy_process_group()


def env_world():
    """(rank, local_rank, world_size, master_addr, master_port) from the torchrun environment."""
    return (int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")),
            int(os.environ.get("WORLD_SIZE", "1")), os.environ.get("MASTER_ADDR", "127.0.0.1"),
            int(os.environ.get("MASTER_PORT", "29500")))


# ---- tree helpers ------------------------------------------------------------------------------------
def broadcast_params(tree, root: int = 0):
    from ..struct import tree as ts
    return ts.tree_map(lambda t: ts._like(t, broadcast(ts._raw(t), root)), tree)


def all_reduce_grads(tree, op: ReduceOp = ReduceOp.avg):
    from ..struct import tree as ts
    return ts.tree_map(lambda t: ts._like(t, all_reduce(ts._raw(t), op)), tree)


def all_reduce_grads_async(tree, op: ReduceOp = ReduceOp.avg):
    """Launch every leaf's all-reduce, then wait for all (Distributed.lean:214-239)."""
    from ..struct import tree as ts
    ls = ts.leaves(tree)
    handles = [all_reduce_async(ts._raw(t), op) for t in ls]
    outs = wait_all(handles)
    return ts.with_leaves(tree, [ts._like(t, o) for t, o in zip(ls, outs)])


def check_all_ranks_healthy(local_ok: bool, device=None) -> bool:
    """Every rank all-reduces(max) a failure flag so all ranks agree
    (Examples/NanoChat/ModdedTrain.lean:1626-1637)."""
    if not is_initialized() or get_world_size() <= 1:
        return local_ok
    flag = torch.tensor([0.0 if local_ok else 1.0], device=device or "cpu")
    return float(all_reduce(flag, ReduceOp.max)[0]) == 0.0
