"""ActorGroup: N actors driven from one process through ``execute_all`` / ``execute_all_async``.

Public surface of the reference (python/ray/actor_group.py:11-221): ``ActorGroup(config, actor_cls,
num_actors, collocate, placement_group_handle)``, ``execute_all``, ``execute_all_async`` with the
same argument rule: if EVERY positional and keyword argument is a list of length ``num_actors`` the
lists are scattered one element per actor, otherwise all arguments are broadcast.

What is different underneath: collocation puts actor i of the vision group and actor i of the text
group in ONE host process per GPU (shared CUDA context, shared ``torch.distributed`` world) instead
of two processes holding half a GPU each, so the vision->text handoff needs no IPC.  A "placement
group" is therefore a pool of host processes; the second group reuses the pool of the first.
Hosts are Ray actors when ``ray`` is importable and requested, else ``multiprocessing`` (spawn)
children speaking a small pipe protocol.  Results stay in the host's object table; the driver holds
:class:`ObjectRef` handles and passes them to later calls, which resolve them locally when the
consumer lives on the same host.

Failure detection lives here, on the host side only: a host that dies closes its pipe (``ActorDiedError``),
a call that exceeds its deadline raises ``ActorTimeoutError``, and every wait polls process liveness.
"""
from __future__ import annotations

import itertools
import logging
import multiprocessing as mp
import os
import time
import traceback
from dataclasses import dataclass

from . import utils
from .actor import TorchDistributedConfig
from .logger import setup_logging

log = logging.getLogger("mmt_b200")


class ActorDiedError(RuntimeError):
    pass


class ActorTimeoutError(TimeoutError):
    pass


class RemoteError(RuntimeError):
    pass


@dataclass(frozen=True)
class ObjectRef:
    host: int
    obj_id: int
    pool_id: int = 0


def _to_cpu(obj):
    """Make a result picklable for the trip to the driver (device tensors become CPU tensors).

    A dict that carries a ``loss_async`` handle (``engine.LossHandle``: the loss was copied to pinned host memory
    behind the step, with an event) is resolved through the handle: waiting for that one event does not drain the
    launch queue, whereas ``loss.cpu()`` would wait for everything the process has enqueued since."""
    import torch
    if isinstance(obj, torch.Tensor):
        return obj.detach().cpu()
    if isinstance(obj, dict):
        handle = obj.get("loss_async")
        if handle is not None and hasattr(handle, "value"):
            out = {k: _to_cpu(v) for k, v in obj.items() if k not in ("loss", "loss_async")}
            out["loss"] = torch.tensor(handle.value())
            return out
        return {k: _to_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_to_cpu(v) for v in obj)
    return obj


class _Host:
    """State of one host process: actors by group id and an object table."""

    def __init__(self, index: int):
        self.index = index
        self.actors: dict[int, object] = {}
        self.objects: dict[int, object] = {}

    def resolve(self, obj):
        if isinstance(obj, ObjectRef):
            if obj.host != self.index:
                raise RemoteError(f"ObjectRef of host {obj.host} cannot be resolved on host {self.index}")
            val = self.objects[obj.obj_id]
            if isinstance(val, BaseException):
                raise val
            return val
        if isinstance(obj, (list, tuple)):
            return type(obj)(self.resolve(v) for v in obj)
        if isinstance(obj, dict):
            return {k: self.resolve(v) for k, v in obj.items()}
        return obj

    def handle(self, msg):
        kind = msg[0]
        if kind == "create":
            _, gid, cls, config, rank = msg
            self.actors[gid] = cls(config, rank)
            return True
        if kind == "call":
            _, gid, method, args, kwargs, oid = msg
            try:
                res = getattr(self.actors[gid], method)(*self.resolve(args), **self.resolve(kwargs))
            except BaseException as e:  # kept in the table so that dependants and fetches re-raise it
                res = RemoteError(f"{type(e).__name__}: {e}\n{traceback.format_exc()}")
                self.objects[oid] = res
                raise res
            self.objects[oid] = res
            return True
        if kind == "put":
            _, oid, value = msg
            self.objects[oid] = value
            return True
        if kind == "fetch":
            val = self.objects[msg[1]]
            if isinstance(val, BaseException):
                raise val
            return _to_cpu(val)
        if kind == "free":
            for oid in msg[1]:
                self.objects.pop(oid, None)
            return True
        if kind == "env":
            os.environ.update({k: str(v) for k, v in msg[1].items()})
            return True
        raise RemoteError(f"unknown message {kind}")


def _host_main(index: int, conn, env: dict):
    os.environ.update(env)
    setup_logging()
    host = _Host(index)
    while True:
        try:
            msg = conn.recv()
        except (EOFError, OSError):
            break
        if msg[0] == "shutdown":
            conn.send((msg[1], True, None))
            break
        seq = msg[1]
        try:
            out = host.handle(msg[2])
            conn.send((seq, True, out))
        except BaseException as e:
            conn.send((seq, False, f"{type(e).__name__}: {e}"))
    try:
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()
    except Exception:
        pass


_POOL_IDS = itertools.count(1)


class HostPool:
    """The builtin "placement group": one spawned host process per bundle (= per GPU)."""

    def __init__(self, num_hosts: int, env: dict | None = None, rpc_timeout_s: float | None = None):
        self.pool_id = next(_POOL_IDS)
        self.num_hosts = num_hosts
        self.rpc_timeout_s = rpc_timeout_s
        ctx = mp.get_context("spawn")
        self.procs, self.conns = [], []
        self._seq = itertools.count(1)
        self._oid = itertools.count(1)
        self._gid = itertools.count(1)
        self._replies: list[dict] = [dict() for _ in range(num_hosts)]
        self.dist_configured = False
        base_env = utils.prepare_runtime_environment()
        base_env.update(env or {})
        for i in range(num_hosts):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=_host_main, args=(i, child, base_env), daemon=True, name=f"mmt-host-{i}")
            p.start()
            child.close()
            self.procs.append(p)
            self.conns.append(parent)

    # -- messaging ------------------------------------------------------------------------
    def send(self, host: int, payload) -> int:
        seq = next(self._seq)
        try:
            self.conns[host].send(("msg", seq, payload))
        except (BrokenPipeError, OSError) as e:
            raise ActorDiedError(f"host {host} is gone: {e}") from e
        return seq

    def wait(self, host: int, seq: int, timeout_s: float | None = None):
        timeout_s = self.rpc_timeout_s if timeout_s is None else timeout_s
        deadline = None if timeout_s is None else time.monotonic() + timeout_s
        conn, replies = self.conns[host], self._replies[host]
        while seq not in replies:
            try:
                ready = conn.poll(0.2)
            except (OSError, EOFError) as e:
                raise ActorDiedError(f"host {host} is gone: {e}") from e
            if ready:
                try:
                    s, ok, val = conn.recv()
                except (EOFError, OSError) as e:
                    raise ActorDiedError(f"host {host} died (pipe closed)") from e
                replies[s] = (ok, val)
            elif not self.procs[host].is_alive():
                raise ActorDiedError(f"host {host} died with exit code {self.procs[host].exitcode}")
            elif deadline is not None and time.monotonic() > deadline:
                raise ActorTimeoutError(f"host {host} did not answer within {timeout_s}s")
        ok, val = replies.pop(seq)
        if not ok:
            raise RemoteError(f"host {host}: {val}")
        return val

    def new_object_id(self) -> int:
        return next(self._oid)

    def new_group_id(self) -> int:
        return next(self._gid)

    def shutdown(self) -> None:
        for i, c in enumerate(self.conns):
            try:
                c.send(("shutdown", 0))
            except Exception:
                pass
        for p in self.procs:
            p.join(timeout=10)
            if p.is_alive():
                p.terminate()
        self.conns, self.procs = [], []


class _PendingRef:
    """An ObjectRef whose producing call may still be running."""

    def __init__(self, pool: HostPool, ref: ObjectRef, seq: int):
        self.pool, self.ref, self.seq, self.done = pool, ref, seq, False

    def wait(self, timeout_s=None):
        if not self.done:
            self.pool.wait(self.ref.host, self.seq, timeout_s)
            self.done = True
        return self.ref


def get(refs, timeout_s: float | None = None):
    """Block for results (a single pending ref or a list), like ``ray.get``."""
    single = not isinstance(refs, (list, tuple))
    items = [refs] if single else list(refs)
    out = []
    for r in items:
        if isinstance(r, _PendingRef):
            ref = r.wait(timeout_s)
            seq = r.pool.send(ref.host, ("fetch", ref.obj_id))
            out.append(r.pool.wait(ref.host, seq, timeout_s))
        else:
            out.append(r)
    return out[0] if single else out


class ActorGroup:
    def __init__(self, config: dict, actor_cls, num_actors: int, collocate: bool = False,
                 placement_group_handle: HostPool | None = None, backend: str | None = None,
                 rpc_timeout_s: float | None = None, env: dict | None = None, gpu_offset: int = 0):
        self.config = config
        self.gpu_offset = int(gpu_offset)      # actor i drives GPU i + gpu_offset (a group on GPUs of its own)
        self.actor_cls = actor_cls
        self.num_actors = num_actors
        self.collocate = collocate
        runtime = utils.select_runtime(str(config.get("runtime", "auto")))
        if placement_group_handle is not None:
            if placement_group_handle.num_hosts != num_actors:
                raise ValueError("the placement group was created for a different number of actors")
            self.pool = placement_group_handle
        elif runtime == "ray":
            from .ray_backend import RayHostPool
            self.pool = RayHostPool(num_actors, env=env, rpc_timeout_s=rpc_timeout_s,
                                    use_gpu=self._default_backend() == "nccl")
        else:
            self.pool = HostPool(num_actors, env=env, rpc_timeout_s=rpc_timeout_s)
        self.placement_group_handle = self.pool
        self.gid = self.pool.new_group_id()
        self.backend = backend or config.get("backend") or self._default_backend()
        seqs = [self.pool.send(i, ("create", self.gid, actor_cls, config, i)) for i in range(num_actors)]
        for i, s in enumerate(seqs):
            self.pool.wait(i, s, timeout_s=600.0)     # process start-up and imports, not an RPC
        saved, self.pool.rpc_timeout_s = self.pool.rpc_timeout_s, None
        try:
            self._setup_process_group()
        finally:
            self.pool.rpc_timeout_s = saved

    @staticmethod
    def _default_backend() -> str:
        try:
            import torch
            return "nccl" if torch.cuda.is_available() else "gloo"
        except Exception:
            return "gloo"

    def _setup_process_group(self) -> None:
        """Rank 0's address and a free port become the rendezvous; every actor gets a torchrun-style env.
        Collocated groups share the hosts and therefore one world: only the first group configures it."""
        if self.pool.dist_configured:
            return
        ips = self.execute_all("get_node_ip_addr")
        ports = self.execute_all("get_free_port")
        cfgs = [TorchDistributedConfig(rank=i, local_rank=i + self.gpu_offset, world_size=self.num_actors,
                                       local_world_size=self.num_actors, master_addr=ips[0], master_port=ports[0],
                                       backend=self.backend) for i in range(self.num_actors)]
        self.execute_all("setup_env_variables", cfgs)
        self.pool.dist_configured = True

    # -- the reference's calling convention ------------------------------------------------
    def _should_scatter(self, args, kwargs) -> bool:
        vals = list(args) + list(kwargs.values())
        return bool(vals) and all(isinstance(v, list) and len(v) == self.num_actors for v in vals)

    def execute_all_async(self, method_name: str, *args, **kwargs) -> list:
        scatter = self._should_scatter(args, kwargs)
        refs = []
        for i in range(self.num_actors):
            a = tuple(v[i] for v in args) if scatter else args
            k = {key: v[i] for key, v in kwargs.items()} if scatter else kwargs
            a, k = self._localise(i, a), self._localise(i, k)
            oid = self.pool.new_object_id()
            seq = self.pool.send(i, ("call", self.gid, method_name, a, k, oid))
            refs.append(_PendingRef(self.pool, ObjectRef(i, oid, self.pool.pool_id), seq))
        return refs

    def execute_all(self, method_name: str, *args, **kwargs) -> list:
        return get(self.execute_all_async(method_name, *args, **kwargs))

    def _localise(self, host: int, obj):
        """Pending refs become plain ObjectRefs for the consumer; a ref living on another host is fetched by the
        driver and shipped by value (the non-collocated path)."""
        if isinstance(obj, _PendingRef):
            ref = obj.ref
            if ref.host == host and ref.pool_id == self.pool.pool_id:
                return ref      # same host: commands run in order, so the value exists when the call runs
            value = get(obj)
            oid = self.pool.new_object_id()
            self.pool.wait(host, self.pool.send(host, ("put", oid, value)))
            return ObjectRef(host, oid, self.pool.pool_id)
        if isinstance(obj, (list, tuple)):
            return type(obj)(self._localise(host, v) for v in obj)
        if isinstance(obj, dict):
            return {k: self._localise(host, v) for k, v in obj.items()}
        return obj

    def free(self, refs) -> None:
        by_host: dict[int, list[int]] = {}
        for r in refs:
            ref = r.ref if isinstance(r, _PendingRef) else r
            if isinstance(ref, ObjectRef):
                by_host.setdefault(ref.host, []).append(ref.obj_id)
        for h, ids in by_host.items():
            self.pool.send(h, ("free", ids))

    def shutdown(self) -> None:
        self.pool.shutdown()
