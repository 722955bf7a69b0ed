"""Data-parallel plumbing: the mirror of Lux's `DistributedUtils` for the one exchange step the
hot path has — all-reduce(avg) of parameter gradients (src/distributed/public_api.jl:270-278 →
ext/MPINCCLExt.jl:71-77).

One process per GPU, launched by torchrun; `torch.distributed` (NCCL over NVLink/NVSwitch on
device tensors, gloo for host tensors) plays the role NCCL.jl + MPI.jl play in the reference.
On top of the reference's per-leaf all-reduce there is a bucketed variant: gradients are packed
into one flat buffer per dtype and reduced with a single collective (per-launch latency, not
link bandwidth, dominates 62 small leaves on NVSwitch).
"""
from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Any, Callable, Sequence

import torch
import torch.distributed as dist


class NCCLBackend:
    """Device tensors over NCCL (ext/MPINCCLExt.jl); host tensors fall back to the wrapped
    host backend exactly like `NCCLBackend` falls back to its `mpi_backend` (:40-54,79-84)."""
    name = "nccl"


class GlooBackend:
    """Host-memory backend (stands where `MPIBackend`, ext/MPIExt.jl, stands in the reference)."""
    name = "gloo"


_state = {"initialized": False, "backend": None, "host_group": None}


def initialized(backend=None) -> bool:
    return _state["initialized"]


def initialize(backend=NCCLBackend, *, timeout_s: float = 600.0, force: bool = False):
    """DistributedUtils.initialize (src/distributed/public_api.jl:20-47): start the process group
    from the launcher's environment (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT, LOCAL_RANK) and
    bind this rank to GPU `local_rank % device_count` (lib/MLDataDevices/ext/CUDAExt.jl:48-51)."""
    if _state["initialized"] and not force:
        return
    import datetime
    name = backend.name if not isinstance(backend, str) else backend
    if name == "nccl":
        if not torch.cuda.is_available():
            raise RuntimeError("NCCLBackend needs CUDA devices")
        local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
        torch.cuda.set_device(local % torch.cuda.device_count())
    if not dist.is_initialized():
        dist.init_process_group(name, timeout=datetime.timedelta(seconds=timeout_s))
    _state.update(initialized=True, backend=name)
    if name == "nccl":  # host arrays travel over a gloo group, as CPU arrays travel over MPI in the reference
        _state["host_group"] = dist.new_group(backend="gloo")


def get_distributed_backend(backend=NCCLBackend):
    if not _state["initialized"]:
        raise RuntimeError("call DistributedUtils.initialize first")
    return backend() if isinstance(backend, type) else backend


def local_rank(backend=None) -> int:
    return dist.get_rank()


def total_workers(backend=None) -> int:
    return dist.get_world_size()


def _group_for(t: torch.Tensor):
    if _state["backend"] == "nccl" and not t.is_cuda:
        return _state["host_group"]
    return None


avg = "avg"


def _wire(t: torch.Tensor) -> torch.Tensor:
    """A contiguous view of the same memory for the collective: column-major (Julia-layout) arrays are
    handed over as their reversed-axes view, everything else must already be contiguous."""
    if t.is_contiguous():
        return t
    r = t.permute(*reversed(range(t.dim())))
    if r.is_contiguous():
        return r
    raise ValueError("collectives need a dense array (column-major or row-major)")

_OPS = {"+": dist.ReduceOp.SUM, "sum": dist.ReduceOp.SUM, "*": dist.ReduceOp.PRODUCT, "prod": dist.ReduceOp.PRODUCT,
        "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}


def bcast_(backend, sendrecvbuf: torch.Tensor, *, root: int = 0) -> torch.Tensor:
    """bcast! (public_api.jl:92-117)."""
    dist.broadcast(_wire(sendrecvbuf), src=root, group=_group_for(sendrecvbuf))
    return sendrecvbuf


def allreduce_(backend, sendrecvbuf: torch.Tensor, op=avg) -> torch.Tensor:
    """allreduce! (public_api.jl:119-152). `avg` maps to NCCL's native average on device tensors
    (ext/MPINCCLExt.jl:74) and to sum followed by a division on host tensors (ext/MPIExt.jl:108-128)."""
    g = _group_for(sendrecvbuf)
    if op == avg:
        if sendrecvbuf.is_cuda and _state["backend"] == "nccl":
            dist.all_reduce(_wire(sendrecvbuf), op=dist.ReduceOp.AVG, group=g)
        else:
            dist.all_reduce(_wire(sendrecvbuf), op=dist.ReduceOp.SUM, group=g)
            sendrecvbuf.div_(dist.get_world_size())
        return sendrecvbuf
    dist.all_reduce(_wire(sendrecvbuf), op=_OPS[op], group=g)
    return sendrecvbuf


def reduce_(backend, sendrecvbuf: torch.Tensor, op="+", *, root: int = 0) -> torch.Tensor:
    """reduce! (public_api.jl:154-188): result valid on `root` only."""
    g = _group_for(sendrecvbuf)
    if op == avg:
        dist.reduce(_wire(sendrecvbuf), dst=root, op=dist.ReduceOp.SUM, group=g)
        if dist.get_rank() == root:
            sendrecvbuf.div_(dist.get_world_size())
        return sendrecvbuf
    dist.reduce(_wire(sendrecvbuf), dst=root, op=_OPS[op], group=g)
    return sendrecvbuf


def synchronize(backend, ps: Any, *, root: int = 0) -> Any:
    """synchronize!! (public_api.jl:197-226, 280-284): broadcast every array / number leaf of a nested
    structure from `root`; anything else (strings, None, symbols) is returned unchanged."""
    if isinstance(ps, torch.Tensor):
        return bcast_(backend, ps, root=root)
    if isinstance(ps, dict):
        return {k: synchronize(backend, v, root=root) for k, v in ps.items()}
    if isinstance(ps, tuple) and hasattr(ps, "_fields"):  # namedtuple
        return type(ps)(*(synchronize(backend, v, root=root) for v in ps))
    if isinstance(ps, (tuple, list)):
        return type(ps)(synchronize(backend, v, root=root) for v in ps)
    if isinstance(ps, bool):
        t = torch.tensor([int(ps)])
        return bool(bcast_(backend, t, root=root).item())
    if isinstance(ps, (int, float)):
        t = torch.tensor([ps], dtype=torch.float64 if isinstance(ps, float) else torch.int64)
        return type(ps)(bcast_(backend, t, root=root).item())
    return ps


class DistributedDataContainer:
    """Contiguous-block shard of a dataset (ext/MLUtilsExt.jl:9-20): ceil(n / workers) consecutive
    indices per rank; the last rank may get fewer."""

    def __init__(self, backend, data, *, rank: int | None = None, workers: int | None = None):
        total = len(data)
        workers = total_workers(backend) if workers is None else workers
        rank = local_rank(backend) if rank is None else rank
        per = int(math.ceil(total / workers)) if total else 0
        lo = min(rank * per, total)
        self.data, self.idxs = data, list(range(lo, min(lo + per, total)))

    def __len__(self):
        return len(self.idxs)

    def __getitem__(self, i):
        return self.data[self.idxs[i]]


@dataclass
class DistributedOptimizer:
    """DistributedOptimizer (public_api.jl:270-278): averages each gradient leaf across the workers
    before delegating to the wrapped rule. `rule(state, param, grad) -> (state, update)`.

    `bucketed=True` reduces all leaves of one dtype in a single flat collective."""
    backend: Any
    rule: Callable
    bucketed: bool = False

    def apply(self, state, param: torch.Tensor, grad: torch.Tensor):
        allreduce_(self.backend, grad, avg)
        return self.rule(state, param, grad)

    def apply_all(self, states: Sequence, params: Sequence[torch.Tensor], grads: Sequence[torch.Tensor]):
        if self.bucketed:
            allreduce_bucketed_(self.backend, list(grads))
            return [self.rule(s, p, g) for s, p, g in zip(states, params, grads)]
        return [self.apply(s, p, g) for s, p, g in zip(states, params, grads)]


def allreduce_bucketed_(backend, grads: Sequence[torch.Tensor], op=avg, bucket_bytes: int = 64 << 20):
    """All-reduce many gradient leaves with one collective per (dtype, device) bucket: pack → reduce →
    unpack. Same result as the per-leaf loop of public_api.jl:275-278 (sums are element-wise)."""
    groups: dict = {}
    for g in grads:
        groups.setdefault((g.dtype, g.device), []).append(g)
    for leaves in groups.values():
        start = 0
        while start < len(leaves):
            size, end = 0, start
            while end < len(leaves) and (end == start or size + leaves[end].numel() * leaves[end].element_size() <= bucket_bytes):
                size += leaves[end].numel() * leaves[end].element_size()
                end += 1
            chunk = leaves[start:end]
            flat = torch.cat([t.reshape(-1) for t in chunk])
            allreduce_(backend, flat, op)
            off = 0
            for t in chunk:
                n = t.numel()
                t.copy_(flat[off:off + n].view_as(t))
                off += n
            start = end
    return grads


class FusedOptimizer:
    """The leaf loop of `Optimisers.update!` under `DistributedOptimizer`
    (src/distributed/public_api.jl:270-278, src/helpers/training.jl:241-245) with one collective and one
    optimiser launch per bucket: gradients of a bucket are summed across the workers in one flat
    all-reduce, then `lb2_optimizer_step` updates every leaf of the bucket with the 1/world averaging
    folded into the step. Rules: "descent", "momentum", "adam" (Optimisers.jl 0.4.6 definitions); state
    arrays have the parameter's dtype; `master=True` keeps an fp32 master copy of bf16 parameters."""

    RULES = {"descent": 0, "momentum": 1, "adam": 2}

    def __init__(self, backend, rule: str = "adam", eta: float = 1e-3, rho: float = 0.9, beta=(0.9, 0.999),
                 eps: float = 1e-8, master: bool = False, bucket_bytes: int = 64 << 20):
        if rule not in self.RULES:
            raise ValueError(f"unknown rule {rule!r}")
        self.backend, self.rule, self.eta, self.rho, self.beta, self.eps = backend, rule, eta, rho, beta, eps
        self.master, self.bucket_bytes = master, bucket_bytes
        self.step_count = 0

    def init(self, params: Sequence[torch.Tensor]):
        """Optimisers.init per leaf."""
        states = []
        for p in params:
            s1 = torch.zeros_like(p) if self.rule in ("momentum", "adam") else None
            s2 = torch.zeros_like(p) if self.rule == "adam" else None
            m = p.detach().to(torch.float32).clone() if (self.master and p.dtype != torch.float32) else None
            states.append((s1, s2, m))
        return states

    def buckets(self, params: Sequence[torch.Tensor]):
        """Leaf indices grouped by (dtype, device), split at bucket_bytes (order preserved)."""
        groups: dict = {}
        for i, p in enumerate(params):
            groups.setdefault((p.dtype, p.device), []).append(i)
        out = []
        for idxs in groups.values():
            cur, size = [], 0
            for i in idxs:
                nbytes = params[i].numel() * params[i].element_size()
                if cur and size + nbytes > self.bucket_bytes:
                    out.append(cur)
                    cur, size = [], 0
                cur.append(i)
                size += nbytes
            if cur:
                out.append(cur)
        return out

    def update(self, states, params: Sequence[torch.Tensor], grads: Sequence[torch.Tensor]):
        """In-place update of params and states from local gradients; returns states."""
        from . import _cabi
        from .arrays import current_stream, dtype_code
        lib = _cabi.load()
        world = total_workers(self.backend) if initialized() else 1
        self.step_count += 1
        for idxs in self.buckets(params):
            chunk = [grads[i] for i in idxs]
            if world > 1:
                flat = torch.cat([_wire(t).reshape(-1) for t in chunk])
                allreduce_(self.backend, flat, "sum")
                views, off = [], 0
                for t in chunk:
                    views.append(flat[off:off + t.numel()])
                    off += t.numel()
            else:
                views = [_wire(t).reshape(-1) for t in chunk]
            leaves = (_cabi.OptLeaf * len(idxs))()
            keep = []
            for k, i in enumerate(idxs):
                p = params[i]
                pw = _wire(p)
                if pw.data_ptr() != p.data_ptr() or not pw.is_contiguous():
                    raise ValueError("parameters must be dense (column- or row-major contiguous)")
                s1, s2, m = states[i]
                gv = views[k] if views[k].is_contiguous() else views[k].contiguous()
                keep.append(gv)
                leaves[k].param = p.data_ptr()
                leaves[k].grad = gv.data_ptr()
                leaves[k].state1 = s1.data_ptr() if s1 is not None else None
                leaves[k].state2 = s2.data_ptr() if s2 is not None else None
                leaves[k].master = m.data_ptr() if m is not None else None
                leaves[k].n = p.numel()
            p0 = params[idxs[0]]
            first = self.rho if self.rule == "momentum" else self.beta[0]
            _cabi.check(lib.lb2_optimizer_step(leaves, len(idxs), self.RULES[self.rule], float(self.eta), float(first),
                                               float(self.beta[1]), float(self.eps), self.step_count, 1.0 / world,
                                               dtype_code(p0.dtype), current_stream(p0.device)))
        return states
