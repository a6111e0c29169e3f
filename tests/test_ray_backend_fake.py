"""The Ray transport of the actor runtime against an in-process stand-in for the ``ray`` module (ray itself is not in
this image).  What is checked is the pool's own contract -- placement group with one bundle per host, one host actor
per bundle, ``send`` returns a ticket, ``wait`` resolves it and maps Ray's timeout / dead-actor / task errors to the
runtime's exception types -- and that an ``ActorGroup`` runs on top of it."""
import sys
import types

import pytest


class _Ticket:
    def __init__(self, value=None, error=None, never=False):
        self.value, self.error, self.never = value, error, never


def _fake_ray():
    ray = types.ModuleType("ray")
    exc = types.ModuleType("ray.exceptions")

    class GetTimeoutError(Exception):
        pass

    class RayActorError(Exception):
        pass

    class RayTaskError(Exception):
        pass

    exc.GetTimeoutError, exc.RayActorError, exc.RayTaskError = GetTimeoutError, RayActorError, RayTaskError
    ray.exceptions = exc
    state = {"init": False, "bundles": None, "options": [], "killed": []}
    ray._state = state
    ray.is_initialized = lambda: state["init"]

    def init(**kw):
        state["init"] = True
    ray.init = init

    class _Method:
        def __init__(self, actor, name):
            self.actor, self.name = actor, name

        def remote(self, *a, **k):
            if self.actor.dead:
                return _Ticket(error=RayActorError("actor died"))
            if self.actor.hang:
                return _Ticket(never=True)
            try:
                return _Ticket(value=getattr(self.actor.obj, self.name)(*a, **k))
            except BaseException as e:          # Ray wraps exceptions of the task
                return _Ticket(error=RayTaskError(f"{type(e).__name__}: {e}"))

    class _Handle:
        def __init__(self, obj):
            self.obj, self.dead, self.hang = obj, False, False

        def __getattr__(self, name):
            return _Method(self, name)

    def remote(cls):
        class _Remote:
            @staticmethod
            def options(**opts):
                state["options"].append(opts)

                class _Bound:
                    @staticmethod
                    def remote(*a, **k):
                        return _Handle(cls(*a, **k))
                return _Bound
        return _Remote
    ray.remote = remote

    def get(ticket, timeout=None):
        if ticket.never:
            raise GetTimeoutError("timeout")
        if ticket.error is not None:
            raise ticket.error
        return ticket.value
    ray.get = get
    ray.kill = lambda h: state["killed"].append(h)

    util = types.ModuleType("ray.util")
    pgm = types.ModuleType("ray.util.placement_group")

    class _PG:
        def ready(self):
            return _Ticket(value=True)

    def placement_group(bundles, strategy="PACK"):
        state["bundles"], state["strategy"] = bundles, strategy
        return _PG()
    pgm.placement_group = placement_group
    ssm = types.ModuleType("ray.util.scheduling_strategies")

    class PlacementGroupSchedulingStrategy:
        def __init__(self, placement_group, placement_group_bundle_index):
            self.pg, self.index = placement_group, placement_group_bundle_index
    ssm.PlacementGroupSchedulingStrategy = PlacementGroupSchedulingStrategy
    util.placement_group, util.scheduling_strategies = pgm, ssm
    ray.util = util
    return {"ray": ray, "ray.exceptions": exc, "ray.util": util, "ray.util.placement_group": pgm,
            "ray.util.scheduling_strategies": ssm}


@pytest.fixture
def fake_ray(monkeypatch):
    mods = _fake_ray()
    for k, v in mods.items():
        monkeypatch.setitem(sys.modules, k, v)
    return mods["ray"]


from multimodal_training_b200.runtime.actor import RayActor  # noqa: E402


class Adder(RayActor):
    def __init__(self, config, rank):
        super().__init__()
        self.base, self.rank = config["base"], rank

    def add(self, x):
        return self.base + self.rank + x

    def boom(self):
        raise ValueError("bad input")


def test_pool_places_one_host_per_bundle_and_maps_ray_errors(fake_ray):
    from multimodal_training_b200.runtime.actor_group import ActorDiedError, ActorTimeoutError, RemoteError
    from multimodal_training_b200.runtime.ray_backend import RayHostPool

    pool = RayHostPool(2, env={"X": "1"}, rpc_timeout_s=1.0, use_gpu=False)
    st = fake_ray._state
    assert st["init"] and st["strategy"] == "PACK" and st["bundles"] == [{"CPU": 6}, {"CPU": 6}]
    assert [o["scheduling_strategy"].index for o in st["options"]] == [0, 1] and "num_gpus" not in st["options"][0]
    assert pool.wait(0, pool.send(0, ("create", 1, Adder, {"base": 10}, 0))) is True
    assert pool.wait(1, pool.send(1, ("create", 1, Adder, {"base": 10}, 1))) is True
    oid = pool.new_object_id()
    assert pool.wait(1, pool.send(1, ("call", 1, "add", (5,), {}, oid))) is True
    assert pool.wait(1, pool.send(1, ("fetch", oid))) == 16
    with pytest.raises(RemoteError, match="bad input"):
        pool.wait(0, pool.send(0, ("call", 1, "boom", (), {}, pool.new_object_id())))
    pool.hosts[0].hang = True
    with pytest.raises(ActorTimeoutError):
        pool.wait(0, pool.send(0, ("fetch", oid)))
    pool.hosts[0].hang, pool.hosts[0].dead = False, True
    with pytest.raises(ActorDiedError):
        pool.wait(0, pool.send(0, ("fetch", oid)))
    pool.shutdown()
    assert len(st["killed"]) == 2 and pool.hosts == []


def test_actor_group_runs_on_the_ray_pool(fake_ray):
    from multimodal_training_b200.runtime.actor_group import ActorGroup

    g = ActorGroup({"base": 100, "runtime": "ray", "device": "cpu"}, Adder, 2)
    assert g.execute_all("add", 1) == [101, 102]
    assert g.execute_all("add", [1, 2]) == [101, 103]          # lists of length num_actors are scattered
    g.shutdown()
