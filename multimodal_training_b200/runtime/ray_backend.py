"""Ray transport for :class:`ActorGroup` hosts (used only when ``ray`` is importable).

One Ray actor per GPU bundle of a PACK placement group ({"GPU": 1, "CPU": 6} per bundle, as in the
reference, python/ray/actor_group.py:52-62) wraps the same host object as the builtin transport, so
the vision and text trainers of a bundle still share one process.  The pool has the interface of
``HostPool``: ``send`` returns a ticket, ``wait`` resolves it.
"""
from __future__ import annotations

import itertools

from . import utils
from .actor_group import ActorDiedError, ActorTimeoutError, RemoteError, _Host


class RayHostPool:
    def __init__(self, num_hosts: int, env: dict | None = None, rpc_timeout_s: float | None = None,
                 use_gpu: bool = True):
        import ray
        from ray.util.placement_group import placement_group
        from ray.util.scheduling_strategies import PlacementGroupSchedulingStrategy

        utils.initialize_ray()
        self.pool_id = id(self) & 0x7fffffff
        self.num_hosts = num_hosts
        self.rpc_timeout_s = rpc_timeout_s
        self.dist_configured = False
        self._seq = itertools.count(1)
        self._oid = itertools.count(1)
        self._gid = itertools.count(1)
        self._tickets: dict[int, object] = {}
        bundle = {"CPU": 6}
        if use_gpu:
            bundle["GPU"] = 1
        self.pg = placement_group([dict(bundle) for _ in range(num_hosts)], strategy="PACK")
        ray.get(self.pg.ready())

        @ray.remote
        class _RayHost:
            def __init__(self, index, env):
                import os
                os.environ.update(env)
                self.host = _Host(index)

            def handle(self, payload):
                return self.host.handle(payload)

        full_env = utils.prepare_runtime_environment()
        full_env.update(env or {})
        self.hosts = []
        for i in range(num_hosts):
            opts = dict(num_cpus=6, scheduling_strategy=PlacementGroupSchedulingStrategy(
                placement_group=self.pg, placement_group_bundle_index=i))
            if use_gpu:
                opts["num_gpus"] = 1
            self.hosts.append(_RayHost.options(**opts).remote(i, full_env))

    def send(self, host: int, payload) -> int:
        seq = next(self._seq)
        self._tickets[seq] = self.hosts[host].handle.remote(payload)
        return seq

    def wait(self, host: int, seq: int, timeout_s: float | None = None):
        import ray
        timeout_s = self.rpc_timeout_s if timeout_s is None else timeout_s
        ticket = self._tickets.pop(seq)
        try:
            return ray.get(ticket, timeout=timeout_s)
        except ray.exceptions.GetTimeoutError as e:
            raise ActorTimeoutError(f"host {host} did not answer within {timeout_s}s") from e
        except ray.exceptions.RayActorError as e:
            raise ActorDiedError(f"host {host} died: {e}") from e
        except ray.exceptions.RayTaskError as e:
            raise RemoteError(f"host {host}: {e}") from e

    def new_object_id(self) -> int:
        return next(self._oid)

    def new_group_id(self) -> int:
        return next(self._gid)

    def shutdown(self) -> None:
        import ray
        for h in self.hosts:
            ray.kill(h)
        self.hosts = []
