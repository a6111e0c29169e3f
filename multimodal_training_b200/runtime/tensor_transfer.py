"""Tensor hand-over between actors (reference: python/ray/tensor_transfer.py:20-282).

Collocated actors of this framework share a process, so the normal path is "local": the tensor
stays where it is and only a key travels.  Two more transports keep the reference's API usable
when actors live in different processes: "ipc" (CUDA IPC handle + interprocess event for two
processes on the SAME physical GPU) and "copy" (host copy, any placement).
"""
from __future__ import annotations

import itertools
from dataclasses import asdict, dataclass, field

import torch

from .utils import get_physical_gpu_id

_LOCAL: dict[int, torch.Tensor] = {}
_KEYS = itertools.count(1)


@dataclass
class TensorTransferRequest:
    transport: str                       # "local" | "ipc" | "copy"
    shape: tuple = ()
    dtype: str = "float32"
    sender_gpu: str = "cpu"
    key: int | None = None               # local
    ipc_handle: tuple | None = None      # ipc: rebuild args from torch.multiprocessing.reductions
    ipc_event: bytes | None = None
    data: object = None                  # copy: CPU tensor
    meta: dict = field(default_factory=dict)

    def to_dict(self) -> dict:
        d = asdict(self)
        d["data"] = self.data
        return d

    @classmethod
    def from_dict(cls, d: dict) -> "TensorTransferRequest":
        return cls(**d)


def create_ipc_handle(t: torch.Tensor):
    """(rebuild args, event handle) for a CUDA tensor; the event marks the producer's stream position."""
    from torch.multiprocessing.reductions import reduce_tensor
    t = t.contiguous()
    ev = torch.cuda.Event(interprocess=True)
    ev.record(torch.cuda.current_stream())
    _, args = reduce_tensor(t)
    return args, ev.ipc_handle()


def reconstruct_tensor_from_ipc(req: TensorTransferRequest) -> torch.Tensor:
    if req.sender_gpu != get_physical_gpu_id():
        raise RuntimeError("CUDA IPC needs sender and receiver on the same physical GPU "
                           f"({req.sender_gpu} vs {get_physical_gpu_id()})")
    from torch.multiprocessing.reductions import rebuild_cuda_tensor
    dev = torch.cuda.current_device()
    ev = torch.cuda.Event.from_ipc_handle(dev, req.ipc_event)
    torch.cuda.current_stream().wait_event(ev)
    args = list(req.ipc_handle)
    args[6] = dev                         # device index of the rebuilt storage
    return rebuild_cuda_tensor(*args)


def prepare_tensor_for_transfer(t: torch.Tensor, receiver_gpu_ids: list[str] | None = None,
                                same_process: bool = True) -> TensorTransferRequest:
    gpu = get_physical_gpu_id() if t.is_cuda else "cpu"
    common = dict(shape=tuple(t.shape), dtype=str(t.dtype).replace("torch.", ""), sender_gpu=gpu)
    if same_process:
        key = next(_KEYS)
        _LOCAL[key] = t
        return TensorTransferRequest("local", key=key, **common)
    if t.is_cuda and receiver_gpu_ids and all(g == gpu for g in receiver_gpu_ids):
        args, ev = create_ipc_handle(t)
        return TensorTransferRequest("ipc", ipc_handle=tuple(args), ipc_event=ev, **common)
    return TensorTransferRequest("copy", data=t.detach().cpu(), **common)


def receive_tensor(req: TensorTransferRequest | dict, device=None) -> torch.Tensor:
    if isinstance(req, dict):
        req = TensorTransferRequest.from_dict(req)
    if req.transport == "local":
        return _LOCAL.pop(req.key)
    if req.transport == "ipc":
        return reconstruct_tensor_from_ipc(req)
    t = req.data
    return t.to(device) if device is not None else t


def gather_gpu_ids(actor_group) -> list[str]:
    return actor_group.execute_all("get_physical_gpu_id")
