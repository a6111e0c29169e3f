"""Trainer base: distributed bring-up, mesh, data source, optimizer policy, step bookkeeping.

One trainer instance is one rank of one model half.  The public surface is the reference's
(python/ray/trainer.py:13-953): ``build_model``, ``initialize_trainer``, ``forward_step``,
``backward_step``, ``optimizer_step``, ``zero_grad``, ``compute_grad_norm_contribution``,
``save_checkpoint``, ``load_checkpoint``, ``get_memory_stats``.  Vision and text trainers that
share a process share the process-wide :class:`ProcessState` (mesh, step contexts, symmetric heap).
"""
from __future__ import annotations

import logging
import os
import random
import time
from dataclasses import dataclass, field

import numpy as np
import torch
import torch.distributed as dist

from ..config.model_configs import VLConfig, get_model_config
from ..data.synthetic import synthetic_global_batch
from ..parallel.mesh import Mesh, build_mesh
from ..parallel.zero import ZeroAdamW, lr_at
from ..runtime.actor import RayActor
from .context import StepContext, build_step_context

log = logging.getLogger("mmt_b200")

DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16,
          "fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}


@dataclass
class ProcessState:
    """What the collocated trainers of one process have in common."""

    mesh: Mesh | None = None
    model_cfg: VLConfig | None = None
    contexts: dict = field(default_factory=dict)
    source: object = None
    heap: object = None           # parallel.symm.SymmetricHeap when fused collectives are on
    fused: object = None


_STATE = ProcessState()


def process_state() -> ProcessState:
    return _STATE


def reset_process_state() -> None:
    global _STATE
    _STATE = ProcessState()


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)


def init_distributed_comm(backend: str | None = None, timeout_s: float | None = None) -> None:
    """``torch.distributed`` from the torchrun-style environment (RANK, WORLD_SIZE, MASTER_ADDR, MASTER_PORT);
    nccl on GPUs, gloo on CPU.  No-op when already initialised or when WORLD_SIZE is 1/unset."""
    if dist.is_initialized():
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1 and "RANK" not in os.environ:
        return
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    kw = {}
    if timeout_s:
        import datetime
        kw["timeout"] = datetime.timedelta(seconds=timeout_s)
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        kw["device_id"] = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    dist.init_process_group(backend=backend, **kw)


def _int_list(v):
    """``[224, 448]`` or ``"224,448"`` (a dotted command-line override) -> list of ints; None stays None."""
    if v is None or v == "":
        return None
    if isinstance(v, str):
        return [int(x) for x in v.replace("[", "").replace("]", "").split(",") if x.strip()]
    if isinstance(v, (int, float)):
        return [int(v)]
    return [int(x) for x in v]


class SyntheticSource:
    """Deterministic global batches of synthetic samples (see ``data/synthetic.py``)."""

    def __init__(self, cfg: VLConfig, global_batch: int, image_size: int, text_tokens: int, seed: int, dtype,
                 pin: bool = False, with_pixels: bool = True, repeat: int = 0, image_sizes=None,
                 text_token_choices=None):
        self.kw = dict(image_size=image_size, text_tokens=text_tokens, seed=seed, dtype=dtype, pin=pin,
                       with_pixels=with_pixels, image_sizes=image_sizes, text_token_choices=text_token_choices)
        self.cfg, self.global_batch, self.repeat = cfg, global_batch, repeat
        self._cache: dict[int, list] = {}

    def global_batch_at(self, step: int) -> list:
        key = step % self.repeat if self.repeat else step
        if key not in self._cache:
            if len(self._cache) > 4 and not self.repeat:
                self._cache.clear()
            self._cache[key] = synthetic_global_batch(self.cfg, key, self.global_batch, **self.kw)
        return self._cache[key]


class Trainer(RayActor):
    kind = "base"

    def __init__(self, config: dict, rank: int = 0):
        super().__init__()
        self.config = dict(config)
        self.rank = rank
        self.seed = int(self.config.get("seed", 42))
        set_seed(self.seed)
        self.model = None
        self.optimizer: ZeroAdamW | None = None
        self.global_step = 0
        self.profile_time = bool(self.config.get("profile_time", False))
        self._last_norm_parts = None

    # ------------------------------------------------------------------ environment
    @property
    def state(self) -> ProcessState:
        return process_state()

    def _get_device(self) -> torch.device:
        if torch.cuda.is_available() and self.config.get("device", "auto") != "cpu":
            return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
        return torch.device("cpu")

    def _dtype(self) -> torch.dtype:
        dt = DTYPES[str(self.config.get("dtype", "bfloat16"))]
        if self._get_device().type == "cuda" and dt != torch.bfloat16:
            raise ValueError("the GPU path computes in bfloat16; set dtype: bfloat16")
        return dt

    def _model_cfg(self) -> VLConfig:
        st = self.state
        if st.model_cfg is None:
            st.model_cfg = get_model_config(self.config.get("model_name", "qwen2_5_vl_7b"))
        return st.model_cfg

    def _ensure_mesh(self) -> Mesh:
        st = self.state
        if st.mesh is None:
            init_distributed_comm(self.config.get("backend"), self.config.get("dist_timeout_s"))
            world = dist.get_world_size() if dist.is_initialized() else 1
            sp = int(self.config.get("mesh_sp", self.config.get("sequence_parallel_size", 1)) or 1)
            tp = int(self.config.get("mesh_tp", self.config.get("tensor_parallel_size", 1)) or 1)
            st.mesh = build_mesh(min(sp, world), min(tp, world))
            if self._get_device().type == "cuda" and st.mesh.world > 1 and self._want_fused_comm():
                from ..parallel import fused as fused_mod
                st.heap, st.fused = fused_mod.try_create(st.mesh, self.config)
        return st.mesh

    def _want_fused_comm(self) -> bool:
        """``training.fused_comm``: true / false / auto.  ``auto`` (the default) means on whenever every GPU of the job
        can address every other one (``parallel.fused.try_create`` checks that and falls back to NCCL otherwise).
        Batches of a data set vary in length; the regions of the symmetric heap are re-reserved per step from sizes
        that are identical on all ranks (``FusedComm.begin_step``) and grow when a longer batch arrives."""
        v = self.config.get("fused_comm", "auto")
        if isinstance(v, str):
            if v.lower() != "auto":
                return v.lower() in ("true", "1", "on", "yes")
            return True
        return bool(v)

    def _ensure_source(self):
        st = self.state
        if st.source is None:
            syn = self.config.get("synthetic")
            cfg = self._model_cfg()
            mesh = self._ensure_mesh()
            if syn:
                gb = int(syn.get("global_batch", int(self.config["batch_size"]) * max(mesh.tdp, 1)))
                st.source = SyntheticSource(cfg, gb, int(syn.get("image_size", 448)), int(syn.get("text_tokens", 64)),
                                            self.seed, torch.bfloat16 if self._get_device().type == "cuda" else
                                            torch.float32, pin=bool(self.config.get("pin_memory", True)),
                                            repeat=int(syn.get("repeat", 0)),
                                            image_sizes=_int_list(syn.get("image_sizes")),
                                            text_token_choices=_int_list(syn.get("text_token_choices")))
            else:
                from ..data.dataset import DatasetSource
                st.source = DatasetSource(self.config, cfg, mesh)
        return st.source

    def step_context(self, step: int) -> StepContext:
        st = self.state
        if step not in st.contexts:
            for k in [k for k in st.contexts if k < step - 1]:
                del st.contexts[k]
            samples = self._ensure_source().global_batch_at(step)
            st.contexts[step] = build_step_context(step, samples, self._model_cfg(), self._ensure_mesh(),
                                                   pad_multiple=self.config.get("pad_multiple"))
        return st.contexts[step]

    # ------------------------------------------------------------------ API shared by both halves
    def initialize_trainer(self) -> bool:
        self._ensure_source()
        return True

    def zero_grad(self, set_to_none: bool = True) -> None:
        if self.optimizer is not None:
            self.optimizer.zero_grad(set_to_none)

    @property
    def accumulation_steps(self) -> int:
        return max(1, int(self.config.get("gradient_accumulation_steps", 1)))

    def data_index(self, step: int, micro: int = 0) -> int:
        """Index of the global batch that micro-step ``micro`` of optimizer step ``step`` consumes."""
        return step * self.accumulation_steps + micro

    def _build_optimizer(self, named_params, group, grad_divisor: float, partial_grad_group=None):
        c = self.config
        # micro-batches of one optimizer step accumulate in the flat gradient; their mean is what AdamW sees
        grad_divisor = grad_divisor * self.accumulation_steps
        self.optimizer = ZeroAdamW(named_params, group=group, lr=float(c.get("learning_rate", 1e-4)),
                                   betas=(float(c.get("adam_beta1", 0.9)), float(c.get("adam_beta2", 0.999))),
                                   eps=float(c.get("adam_eps", 1e-8)), weight_decay=float(c.get("weight_decay", 0.0)),
                                   grad_divisor=grad_divisor, partial_grad_group=partial_grad_group,
                                   fused=self.state.fused,
                                   master_weights=bool(c.get("optimizer_master_weights", True)))
        return self.optimizer

    def _total_steps(self) -> int:
        # the reference sizes the schedule by one epoch (python/ray/vision.py:408); this uses all epochs
        return int(self.config.get("num_iterations", 1)) * int(self.config.get("num_epochs", 1))

    def current_lr(self) -> float:
        c = self.config
        total = self._total_steps()
        warm = int(c.get("warmup_steps", 0))
        if float(c.get("warmup_ratio", 0) or 0) > 0:
            warm = int(float(c["warmup_ratio"]) * total)
        return lr_at(self.global_step, base_lr=float(c.get("learning_rate", 1e-4)), total_steps=total,
                     warmup_steps=warm, kind=str(c.get("lr_scheduler_type", "cosine")))

    def compute_grad_norm_contribution(self) -> dict:
        """Squared-norm pieces of this rank after gradient reduction: ``{"type", "sharded", "replicated"}``.
        The driver combines them with ``aggregate_grad_norms`` (reference: python/train_ray.py:37-122)."""
        opt = self.optimizer
        shard = opt.reduce_gradients()
        self._reduced_shard = shard
        a, b = opt.grad_norm_sq_local(shard)
        self._last_norm_parts = (a, b)
        return {"type": self.norm_type, "sharded": float(a.item()), "replicated": float(b.item()),
                "zero_size": opt.gsize, "zero_rank": opt.grank, "tp_size": self._norm_tp_size()}

    def _norm_tp_size(self) -> int:
        """Size of the group inside which this trainer's replicated parameters repeat."""
        mesh = self._ensure_mesh()
        if self.kind == "vision":
            return mesh.sp if getattr(self, "tensor_parallel", False) else 1
        return mesh.tp

    def optimizer_step(self, global_grad_norm: float | None = None) -> float:
        """Clip (if configured and a global norm is given) -> fused AdamW on the owned shard -> parameter all-gather."""
        c = self.config
        scale = None
        if c.get("clip_grad_norm") and global_grad_norm is not None:
            max_norm = float(c.get("max_grad_norm", 1.0))
            scale = min(1.0, max_norm / (float(global_grad_norm) + 1e-6))
        shard = getattr(self, "_reduced_shard", None)
        self._reduced_shard = None
        lr = self.current_lr()
        self.optimizer.step(lr=lr, grad_scale=scale, shard=shard)
        self.global_step += 1
        if self.kind == "text" and self.state.fused is not None:
            # once per step and process, on the driver's calling thread: after a step that reserved or moved
            # regions of the symmetric heap all ranks compare their layouts (HybridEngine does the same itself)
            self.state.fused.end_step()
        return lr

    def check_device_errors(self) -> bool:
        """Raise if a kernel of this process recorded a bounded wait that ran out (or a skipped out-of-range access)
        since the last check.  Synchronises the device: call it where the host waits anyway."""
        if self._get_device().type == "cuda":
            from ..ops import native as nv
            if nv.available():
                try:
                    nv.raise_on_device_error()
                except RuntimeError:
                    if self.state.fused is not None:
                        self.state.fused.reset_after_error()
                    raise
        return True

    def get_memory_stats(self) -> dict:
        # no device synchronisation here: the driver calls this at its logging points between steps that are still
        # in flight.  Device-side failures reach the driver with the loss (TextTrainer._loss_handle copies the error
        # word behind every forward) and are checked with a synchronisation before every checkpoint.
        if self._get_device().type == "cuda":
            return {"allocated_mb": torch.cuda.memory_allocated() / 2 ** 20,
                    "peak_mb": torch.cuda.max_memory_allocated() / 2 ** 20}
        return {"allocated_mb": 0.0, "peak_mb": 0.0}

    def set_receiver_info(self, *args, **kwargs) -> bool:
        """Kept for API parity: collocated halves share a process here, so no receiver wiring is needed."""
        return True

    def get_rank(self) -> int:
        return self.rank

    def _timer_start(self):
        if self.profile_time:
            if self._get_device().type == "cuda":
                torch.cuda.synchronize()
            return time.perf_counter()
        return None

    def _timer_stop(self, t0):
        if t0 is None:
            return None
        if self._get_device().type == "cuda":
            torch.cuda.synchronize()
        return (time.perf_counter() - t0) * 1e3

    # ------------------------------------------------------------------ checkpoints (reference layout)
    @staticmethod
    def _ckpt_name(epoch) -> str:
        """``epoch`` is an epoch number or the name of a checkpoint directory (``step_120``)."""
        return epoch if isinstance(epoch, str) else f"epoch_{epoch}"

    def _ckpt_path(self, checkpoint_dir: str, epoch) -> str:
        return os.path.join(checkpoint_dir, self._ckpt_name(epoch), self.kind, f"rank_{self.rank}.pt")

    def set_global_step(self, step: int) -> int:
        """Position of the learning-rate schedule after a resume (optimizer steps already done)."""
        self.global_step = int(step)
        return self.global_step

    def save_checkpoint(self, checkpoint_dir: str, epoch) -> str:
        self.check_device_errors()          # never write weights that a failed exchange may have corrupted
        path = self._ckpt_path(checkpoint_dir, epoch)
        os.makedirs(os.path.dirname(path), exist_ok=True)
        payload = {"model": {k: v.cpu() for k, v in self.model.reference_state_dict().items()}}
        tmp = path + ".tmp"
        torch.save(payload, tmp)
        os.replace(tmp, path)
        if self.config.get("save_optimizer", False) and self.optimizer is not None:
            opath = os.path.join(checkpoint_dir, self._ckpt_name(epoch), self.kind + "_optim", f"rank_{self.rank}.pt")
            os.makedirs(os.path.dirname(opath), exist_ok=True)
            extra = {"optimizer": self.optimizer.state_dict(), "global_step": self.global_step,
                     "rng": torch.get_rng_state()}
            torch.save(extra, opath + ".tmp")
            os.replace(opath + ".tmp", opath)
        return path

    def load_checkpoint(self, checkpoint_dir: str, epoch) -> bool:
        """Load this rank's shard; False if it is missing or unreadable.  On failure the weights this trainer had
        before the call are put back (a partial load must not leave some tensors from the checkpoint and others from
        the initialisation) and the caller decides for ALL ranks together whether training starts from scratch."""
        path = self._ckpt_path(checkpoint_dir, epoch)
        if not os.path.exists(path):
            log.warning("checkpoint %s not found", path)
            return False
        backup = {k: v.detach().clone() for k, v in self.model.state_dict().items()}
        try:
            payload = torch.load(path, map_location="cpu", weights_only=True)
            self._load_model_state(payload["model"], sharded=True)
            if self.optimizer is not None:
                self.optimizer.refresh_master_from_params()
                opath = os.path.join(checkpoint_dir, self._ckpt_name(epoch), self.kind + "_optim",
                                     f"rank_{self.rank}.pt")
                if os.path.exists(opath):
                    extra = torch.load(opath, map_location="cpu", weights_only=True)
                    self.optimizer.load_state_dict(extra["optimizer"])
                    self.global_step = int(extra.get("global_step", self.global_step))
                    if extra.get("rng") is not None:
                        torch.set_rng_state(extra["rng"].cpu().to(torch.uint8))
            return True
        except Exception as e:  # a broken shard must not kill the run (the driver starts from scratch)
            log.error("failed to load checkpoint %s: %s", path, e)
            with torch.no_grad():
                for k, v in self.model.state_dict().items():
                    v.copy_(backup[k])
            if self.optimizer is not None:
                self.optimizer.refresh_master_from_params()
            return False

    def _load_model_state(self, sd: dict, sharded: bool) -> None:
        raise NotImplementedError
