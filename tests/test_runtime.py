"""Actor runtime: ActorGroup calling convention, collocation on shared hosts, object refs, failure detection
(host side only: an actor that raises, a host process that exits, an RPC deadline), logging, tensor transfer,
and the driver loop end to end on CPU (gloo) with checkpoint + resume."""
import logging
import os
import time

import pytest
import torch

from multimodal_training_b200.runtime.actor import RayActor
from multimodal_training_b200.runtime.actor_group import (ActorDiedError, ActorGroup, ActorTimeoutError, RemoteError,
                                                          get)

pytestmark = pytest.mark.integration


class Echo(RayActor):
    def __init__(self, config, rank):
        super().__init__()
        self.config, self.rank, self.store = config, rank, {}

    def whoami(self):
        return {"rank": self.rank, "pid": os.getpid(), "env_rank": os.environ.get("RANK"),
                "world": os.environ.get("WORLD_SIZE"), "port": os.environ.get("MASTER_PORT")}

    def add(self, a, b=0):
        return a + b + self.rank

    def make_tensor(self, n):
        return {"t": torch.full((n,), float(self.rank)), "tag": self.config.get("tag")}

    def consume(self, obj, k):
        return float(obj["t"].sum()) + k

    def boom(self):
        raise ValueError("kaboom")

    def die(self):
        os._exit(3)

    def sleep(self, s):
        time.sleep(s)
        return s


def test_scatter_broadcast_and_shared_world():
    g = ActorGroup({"tag": "a", "runtime": "builtin"}, Echo, 2, backend="gloo")
    try:
        info = g.execute_all("whoami")
        assert [i["rank"] for i in info] == [0, 1] and [i["env_rank"] for i in info] == ["0", "1"]
        assert info[0]["world"] == "2" and info[0]["port"] == info[1]["port"]
        assert g.execute_all("add", 10, b=1) == [11, 12]                 # broadcast
        assert g.execute_all("add", [10, 20], b=[1, 2]) == [11, 23]      # every arg is a list of length N: scatter
        # a list mixed with a scalar is NOT scattered (reference rule): the whole list is broadcast
        with pytest.raises(RemoteError, match="TypeError"):
            g.execute_all("add", [10, 20], b=1)
    finally:
        g.shutdown()


def test_collocated_groups_share_hosts_and_refs_resolve_locally():
    g1 = ActorGroup({"tag": "vision", "runtime": "builtin"}, Echo, 2, collocate=True, backend="gloo")
    g2 = ActorGroup({"tag": "text", "runtime": "builtin"}, Echo, 2, collocate=True,
                    placement_group_handle=g1.placement_group_handle)
    try:
        p1, p2 = g1.execute_all("whoami"), g2.execute_all("whoami")
        assert [a["pid"] for a in p1] == [b["pid"] for b in p2]          # actor i of both groups: one process
        assert p1[0]["port"] == p2[0]["port"]                            # one torch.distributed world
        refs = g1.execute_all_async("make_tensor", 4)
        out = g2.execute_all("consume", refs, [1, 2])                    # refs + list: scattered, resolved on host
        assert out == [1.0, 6.0]
        fetched = get(refs)
        assert fetched[1]["tag"] == "vision" and fetched[1]["t"].tolist() == [1.0] * 4
    finally:
        g1.shutdown()


def test_actor_exception_is_reported_and_the_group_survives():
    g = ActorGroup({"runtime": "builtin"}, Echo, 2, backend="gloo")
    try:
        with pytest.raises(RemoteError, match="kaboom"):
            g.execute_all("boom")
        assert g.execute_all("add", 1) == [1, 2]
    finally:
        g.shutdown()


def test_dead_host_and_rpc_deadline_are_detected():
    g = ActorGroup({"runtime": "builtin"}, Echo, 2, backend="gloo", rpc_timeout_s=1.0)
    try:
        with pytest.raises(ActorTimeoutError):
            g.execute_all("sleep", 3.0)
        time.sleep(2.5)
        refs = g.execute_all_async("die")
        with pytest.raises((ActorDiedError, RemoteError)):
            get(refs, timeout_s=20)
    finally:
        g.shutdown()


def test_tensor_transfer_local_and_copy():
    from multimodal_training_b200.runtime.tensor_transfer import (TensorTransferRequest,
                                                                  prepare_tensor_for_transfer, receive_tensor)
    t = torch.arange(6.0).reshape(2, 3)
    req = prepare_tensor_for_transfer(t)
    assert req.transport == "local" and receive_tensor(req.to_dict()) is t
    req = prepare_tensor_for_transfer(t, receiver_gpu_ids=["cpu"], same_process=False)
    assert req.transport == "copy" and torch.equal(receive_tensor(TensorTransferRequest.from_dict(req.to_dict())), t)


def test_setup_logging_is_idempotent(tmp_path, monkeypatch):
    from multimodal_training_b200.runtime import logger
    monkeypatch.setenv("RAY_TRAIN_LOG_FILE", str(tmp_path / "train.log"))
    root = logger.setup_logging(force=True)
    n = len(root.handlers)
    logger.setup_logging()
    assert len(root.handlers) == n
    logging.getLogger("x").info("hello")
    for h in root.handlers:
        h.flush()
    assert "hello" in (tmp_path / "train.log").read_text()
    logger.setup_logging(force=True, log_file="/tmp/ray_train.log")


def _cfg(tmp_path, **over):
    from multimodal_training_b200.config.loader import load_config
    ov = ["vision.model_name=tiny", "text.model_name=tiny", "vision.dtype=float32", "text.dtype=float32",
          "vision.parallelism=sequence", "text.parallelism=tensor", "training.parallel_size=2",
          "training.batch_size=2", "training.num_iterations=3", "training.num_epochs=1", "training.warmup_steps=1",
          "training.learning_rate=1e-3", "training.warmup_ratio=0", "training.lr_scheduler_type=constant",
          "+training.device=cpu", "training.backend=gloo", "training.runtime=builtin", "training.clip_grad_norm=true",
          "training.no_checkpoint=false", f"training.checkpoint_dir={tmp_path / 'ckpt'}",
          "+data.synthetic.image_size=224", "+data.synthetic.text_tokens=64", "+data.synthetic.global_batch=2",
          "+data.synthetic.repeat=1"]
    return load_config(None, ov + [f"{k}={v}" for k, v in over.items()])


def test_driver_trains_checkpoints_and_resumes(tmp_path, caplog):
    from multimodal_training_b200 import train
    from multimodal_training_b200.checkpoint import find_latest_checkpoint
    res = train.main(_cfg(tmp_path))
    assert res["steps"] == 3 and res["losses"][-1] < res["losses"][0]
    ck = tmp_path / "ckpt"
    assert find_latest_checkpoint(str(ck)) == 0
    for half in ("vision", "text"):
        for r in range(2):
            assert (ck / "epoch_0" / half / f"rank_{r}.pt").exists()
    assert (ck / "epoch_0" / "metadata.json").exists()
    sd = torch.load(ck / "epoch_0" / "text" / "rank_1.pt")["model"]
    assert "layers.0.self_attn.q_proj.weight" in sd and sd["layers.0.mlp.down_proj.weight"].shape == (256, 344)
    # resume: epoch 0 is done, so a 2-epoch run continues at epoch 1 from the saved weights
    res2 = train.main(_cfg(tmp_path, **{"training.num_epochs": 2}))
    assert res2["steps"] == 6 and len(res2["losses"]) == 3
    assert res2["losses"][0] < res["losses"][0]
    assert find_latest_checkpoint(str(ck)) == 1
    log = open("/tmp/ray_train.log").read() if os.path.exists("/tmp/ray_train.log") else ""
    assert "Training completed!" in log and "avg" in log


def test_step_checkpoints_resume_inside_an_epoch(tmp_path):
    """A run that stops inside an epoch continues from its last ``step_S`` checkpoint (weights, optimizer shards, step
    counter, data position) and then produces the losses of a run that was never interrupted."""
    from multimodal_training_b200 import train
    from multimodal_training_b200.checkpoint import find_latest_checkpoint, find_latest_step_checkpoint
    common = {"training.num_iterations": 5, "+data.synthetic.repeat": 0, "+training.save_optimizer": "true",
              "training.lr_scheduler_type": "cosine", "training.warmup_steps": 0}
    whole = train.main(_cfg(tmp_path / "a", **common))
    assert whole["steps"] == 5
    part = dict(common, **{"training.save_every_steps": 2, "training.max_steps": 3})
    first = train.main(_cfg(tmp_path / "b", **part))
    ck = tmp_path / "b" / "ckpt"
    assert first["steps"] == 3 and find_latest_checkpoint(str(ck)) is None
    meta = find_latest_step_checkpoint(str(ck))
    assert meta["global_step"] == 2 and meta["epoch"] == 0 and meta["next_iteration"] == 2
    assert (ck / "step_2" / "text_optim" / "rank_0.pt").exists()
    rest = train.main(_cfg(tmp_path / "b", **dict(common, **{"training.save_every_steps": 2})))
    assert rest["steps"] == 5 and len(rest["losses"]) == 3          # steps 2, 3 and 4 ran again / for the first time
    for a, b in zip(first["losses"], whole["losses"][:3]):
        assert abs(a - b) < 1e-6 * abs(b)
    for a, b in zip(rest["losses"], whole["losses"][2:]):
        assert abs(a - b) < 1e-5 * abs(b), (rest["losses"], whole["losses"])
    # the finished epoch supersedes the step checkpoints; only the newest two of those are kept
    assert find_latest_checkpoint(str(ck)) == 0
    assert sorted(p.name for p in ck.iterdir() if p.name.startswith("step_")) == ["step_2", "step_4"]
    again = train.main(_cfg(tmp_path / "b", **dict(common, **{"training.save_every_steps": 2})))
    assert again["steps"] == 5 and again["losses"] == []            # nothing left to do


def _spmd_worker(rank, world, ckpt_root, over):
    from multimodal_training_b200 import train_spmd
    import pathlib
    return train_spmd.main(_cfg(pathlib.Path(ckpt_root), **over))


def test_spmd_driver_matches_the_actor_driver_and_resumes(tmp_path):
    """The torchrun-style driver trains like the actor driver on the same configuration (same losses), writes the
    same checkpoint layout, and each can resume from the other's checkpoint."""
    from dist_utils import run_ranks
    from multimodal_training_b200 import train
    from multimodal_training_b200.checkpoint import find_latest_checkpoint
    actor = train.main(_cfg(tmp_path / "actor"))
    for d in ("r1", "r2"):
        (tmp_path / d).mkdir()
    spmd = run_ranks(_spmd_worker, 2, tmp_path / "r1", str(tmp_path / "spmd"), {})
    assert spmd[0]["steps"] == 3 and spmd[0]["losses"] == spmd[1]["losses"]
    for a, b in zip(spmd[0]["losses"], actor["losses"]):
        assert abs(a - b) < 1e-6 * abs(b), (spmd[0]["losses"], actor["losses"])
    ck = tmp_path / "spmd" / "ckpt"
    assert find_latest_checkpoint(str(ck)) == 0
    for half in ("vision", "text"):
        for r in range(2):
            assert (ck / "epoch_0" / half / f"rank_{r}.pt").exists()
    # second epoch: the SPMD driver continues from its own checkpoint, the actor driver from the SPMD one
    more = run_ranks(_spmd_worker, 2, tmp_path / "r2", str(tmp_path / "spmd"), {"training.num_epochs": 2})
    assert more[0]["steps"] == 6 and len(more[0]["losses"]) == 3
    import shutil
    shutil.rmtree(ck / "epoch_1")
    cross = train.main(_cfg(tmp_path / "spmd", **{"training.num_epochs": 2}))
    assert cross["steps"] == 6
    for a, b in zip(more[0]["losses"], cross["losses"]):
        assert abs(a - b) < 1e-6 * abs(b)


def test_driver_trains_on_image_files(tmp_path):
    """End to end on real files: PNG images and a LLaVA-style annotation file go through the in-tree processor
    (resize, patch layout, chat template, placeholder expansion, label mask), the sequence-parallel vision encoder,
    the handoff and the tensor-parallel decoder.  The trainers' own guards check that placeholders and vision rows
    agree; here the run has to finish with finite losses and supervise only the answers."""
    import json
    import numpy as np
    from PIL import Image
    from multimodal_training_b200 import train
    from multimodal_training_b200.config.model_configs import get_model_config
    from multimodal_training_b200.data.dataset import default_processor
    from multimodal_training_b200.data.preprocessing import preprocess_qwen_visual
    rng = np.random.default_rng(0)
    ann = []
    for i in range(4):
        Image.fromarray(rng.integers(0, 255, (200 + 10 * i, 260, 3), dtype=np.uint8)).save(tmp_path / f"im{i}.png")
        ann.append({"image": f"im{i}.png", "conversations": [{"from": "human", "value": "<image>\nWhat is shown?"},
                                                             {"from": "gpt", "value": f"Picture number {i}."}]})
    (tmp_path / "ann.json").write_text(json.dumps(ann))
    # one sample by hand: 224 x 224 after the fixed-size resize -> 256 patches, 64 placeholders, answer-only labels
    cfg_m = get_model_config("tiny")
    enc = preprocess_qwen_visual([ann[0]], default_processor("tiny", cfg_m), data_path=str(tmp_path),
                                 max_pixels=224 * 224, min_pixels=224 * 224, force_fixed_size=True)
    assert enc["pixel_values"].shape == (256, 1176) and enc["image_grid_thw"].tolist() == [[1, 16, 16]]
    ids, labels = enc["input_ids"][0], enc["labels"][0]
    assert int((ids == cfg_m.image_token_id).sum()) == 64 and int(ids.max()) < cfg_m.text.vocab_size
    kept = labels[labels != -100]
    assert 0 < kept.numel() < 40 and bytes(int(t) for t in kept if t < 256).decode().startswith("Picture number 0.")
    assert bool((labels[ids == cfg_m.image_token_id] == -100).all())

    from multimodal_training_b200.config.loader import load_config
    ov = ["vision.model_name=tiny", "text.model_name=tiny", "vision.dtype=float32", "text.dtype=float32",
          "vision.parallelism=sequence", "text.parallelism=tensor", "training.parallel_size=2",
          "training.batch_size=2", "training.num_iterations=3", "training.num_epochs=1", "training.warmup_steps=0",
          "training.learning_rate=1e-3", "training.warmup_ratio=0", "training.lr_scheduler_type=constant",
          "+training.device=cpu", "training.backend=gloo", "training.runtime=builtin",
          "data.datasets=[toy]", f"+data.data_registry.toy.annotation_path={tmp_path / 'ann.json'}",
          f"+data.data_registry.toy.data_path={tmp_path}", "data.num_workers=0", "data.pin_memory=false",
          f"data.max_pixels={224 * 224}", f"data.min_pixels={224 * 224}", "data.force_fixed_size=true"]
    res = train.main(load_config(None, ov))
    assert res["steps"] == 3 and all(v == v and v < 20 for v in res["losses"])
    assert res["losses"][-1] < res["losses"][0]          # 4 samples, batch 2: the third step sees step one's data again


@pytest.mark.parametrize("vision_mode", ["sequence", "tensor"])
def test_pretrained_split_train_merge_chain_keeps_the_weights(tmp_path, vision_mode):
    """A full HF-layout checkpoint is split, loaded by sequence-parallel vision and tensor-parallel text trainers
    (``pretrained_checkpoint_dir``), saved as per-rank shards after steps with a vanishing learning rate, merged, and
    loaded into the single-process model: its logits equal the original model's."""
    from multimodal_training_b200 import train
    from multimodal_training_b200.cli import merge_checkpoint, split_checkpoint
    from multimodal_training_b200.models.vlm import Qwen2_5_VLForConditionalGeneration
    src = Qwen2_5_VLForConditionalGeneration("tiny", seed=5)
    full = {"model.visual." + k: v for k, v in src.model.visual.reference_state_dict(fused_qkv=True).items()}
    for k, v in src.model.language_model.reference_state_dict().items():
        full[k if k.startswith("lm_head") else "model.language_model." + k] = v
    torch.save(full, tmp_path / "hf_full.pt")
    split_dir = split_checkpoint.split_checkpoint(str(tmp_path / "hf_full.pt"), str(tmp_path / "split"))
    cfg = _cfg(tmp_path, **{"training.learning_rate": 1e-30, "training.num_iterations": 2,
                            "training.weight_decay": 0.0, "+vision.pretrained_checkpoint_dir": split_dir,
                            "+text.pretrained_checkpoint_dir": split_dir, "vision.parallelism": vision_mode})
    res = train.main(cfg)
    assert res["steps"] == 2
    out = merge_checkpoint.merge_checkpoint(str(tmp_path / "ckpt" / "epoch_0"), str(tmp_path / "merged"), "tiny", 2,
                                            vision_tensor_parallel=vision_mode == "tensor")
    merged = torch.load(os.path.join(out, "pytorch_model.bin"))
    for k, v in full.items():
        key = k[len("model."):] if k.startswith("model.") else k
        assert key in merged, key
        assert merged[key].shape == v.shape, key
        assert torch.allclose(merged[key], v, rtol=0, atol=1e-20), key     # two AdamW steps of size 1e-30
    dst = Qwen2_5_VLForConditionalGeneration("tiny", seed=99)
    dst.load_merged_state_dict(merged)
    cfgm = src.config
    ids = torch.randint(10, 900, (1, 80))
    ids[0, 5] = cfgm.vision_start_token_id
    ids[0, 6:70] = cfgm.image_token_id
    pix = torch.randn(256, cfgm.vision.patch_dim)
    with torch.no_grad():
        assert torch.allclose(dst.model(ids, pix, [(1, 16, 16)]), src.model(ids, pix, [(1, 16, 16)]), atol=1e-5)


def _file_cfg(tmp_path, ann_name, **over):
    from multimodal_training_b200.config.loader import load_config
    ov = ["vision.model_name=tiny", "text.model_name=tiny", "vision.dtype=float32", "text.dtype=float32",
          "vision.parallelism=sequence", "text.parallelism=tensor", "training.parallel_size=2",
          "training.batch_size=2", "training.num_iterations=4", "training.num_epochs=1", "training.warmup_steps=0",
          "training.learning_rate=1e-3", "training.warmup_ratio=0", "training.lr_scheduler_type=constant",
          "training.clip_grad_norm=true", "+training.device=cpu", "training.backend=gloo", "training.runtime=builtin",
          "data.datasets=[toy]", f"+data.data_registry.toy.annotation_path={tmp_path / ann_name}",
          f"+data.data_registry.toy.data_path={tmp_path}", "data.num_workers=0", "data.pin_memory=false",
          "data.force_fixed_size=false", "data.min_pixels=3136", "data.max_pixels=200704"]
    return load_config(None, ov + [f"{k}={v}" for k, v in over.items()])


def test_driver_handles_ragged_multi_image_and_text_only_samples(tmp_path):
    """Images of different sizes and aspect ratios (no fixed-size resize), a sample with two images and a sample
    without any share batches; a data set without a single image trains the decoder alone."""
    import json
    import numpy as np
    from PIL import Image
    from multimodal_training_b200 import train
    rng = np.random.default_rng(1)
    ann = []
    for i, (h, w) in enumerate([(200, 260), (336, 224), (280, 420), (140, 500), (448, 448), (230, 230)]):
        Image.fromarray(rng.integers(0, 255, (h, w, 3), dtype=np.uint8)).save(tmp_path / f"im{i}.png")
        ann.append({"image": f"im{i}.png", "conversations": [{"from": "human", "value": "<image>\nDescribe."},
                                                             {"from": "gpt", "value": f"Image {i}, {h} by {w}."}]})
    ann.append({"image": ["im0.png", "im4.png"], "conversations": [{"from": "human", "value": "<image><image>\nSame?"},
                                                                   {"from": "gpt", "value": "No."}]})
    ann.append({"conversations": [{"from": "human", "value": "Hello?"}, {"from": "gpt", "value": "Hi."}]})
    (tmp_path / "ann.json").write_text(json.dumps(ann))
    # batches prepared ahead on worker threads are the same batches
    from multimodal_training_b200.config.loader import trainer_configs
    from multimodal_training_b200.config.model_configs import get_model_config
    from multimodal_training_b200.data.dataset import DatasetSource
    from multimodal_training_b200.parallel.mesh import Mesh
    sources = [DatasetSource(trainer_configs(_file_cfg(tmp_path, "ann.json", **{"data.num_workers": w}))[1],
                             get_model_config("tiny"), Mesh()) for w in (0, 2)]
    for step in (0, 1, 3):                                           # step 2 is skipped on purpose
        for a, b in zip(sources[0].global_batch_at(step), sources[1].global_batch_at(step)):
            assert torch.equal(a.input_ids, b.input_ids) and torch.equal(a.labels, b.labels)
            assert a.grid_thw == b.grid_thw and a.sample_index == b.sample_index
            assert (a.pixel_values is None) == (b.pixel_values is None)
            assert a.pixel_values is None or torch.equal(a.pixel_values, b.pixel_values)
    res = train.main(_file_cfg(tmp_path, "ann.json", **{"data.num_workers": 2}))   # 4 steps x 2: every sample once
    assert res["steps"] == 4 and all(v == v and v < 20 for v in res["losses"])
    # text tensor parallel off, two data-parallel text replicas with one sample each (with and without images)
    res = train.main(_file_cfg(tmp_path, "ann.json", **{"text.parallelism": "none", "training.batch_size": 1}))
    assert res["steps"] == 4 and all(v == v and v < 20 for v in res["losses"])
    text_only = [{"conversations": [{"from": "human", "value": f"Hello {i}?"}, {"from": "gpt", "value": f"Hi {i}."}]}
                 for i in range(4)]
    (tmp_path / "text.json").write_text(json.dumps(text_only))
    res = train.main(_file_cfg(tmp_path, "text.json", **{"training.num_iterations": 2}))
    assert res["steps"] == 2 and res["losses"][1] < res["losses"][0]


def _lossy_spmd_worker(rank, world, root):
    """Rank 1 leaves after the first step (between steps, nothing of its own in flight); rank 0 must get an error
    from its next collective instead of waiting forever."""
    import pathlib
    import torch.distributed as dist
    from multimodal_training_b200.engine import HybridEngine
    eng = HybridEngine.from_config(_cfg(pathlib.Path(root)))
    first = float(eng.train_step(0))
    dist.barrier()
    if rank == 1:
        os._exit(0)
    import json
    t0 = time.time()
    try:
        eng.train_step(1)
        out = {"first": first, "error": None, "waited": time.time() - t0}
    except Exception as e:      # gloo reports the closed connection
        out = {"first": first, "error": type(e).__name__, "waited": time.time() - t0}
    with open(os.path.join(root, "survivor.json"), "w") as f:       # the harness's own final barrier fails too
        json.dump(out, f)
    return out


def test_a_rank_that_leaves_between_steps_fails_the_others_next_collective(tmp_path):
    import torch.multiprocessing as mp
    from dist_utils import _entry, free_port
    port = free_port()
    (tmp_path / "c").mkdir()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_entry, args=(r, 2, port, _lossy_spmd_worker, (str(tmp_path / "c"),), str(tmp_path)))
             for r in range(2)]
    for p in procs:
        p.start()
    procs[0].join(180)
    alive = procs[0].is_alive()
    for p in procs:
        if p.is_alive():
            p.terminate()
    assert not alive, "rank 0 is still waiting for the rank that left"
    import json
    res = json.load(open(tmp_path / "c" / "survivor.json"))
    assert res["error"] is not None and res["waited"] < 120 and res["first"] == res["first"], res


def test_non_collocated_groups_train_like_collocated_ones(tmp_path):
    """``training.collocate: false``: the text actors live in host processes (and a torch.distributed world) of their
    own; vision rows and their gradients travel between the groups by value through the driver.  Same losses as
    the collocated run, and the two groups really are different processes."""
    from multimodal_training_b200 import train
    from multimodal_training_b200.runtime.actor_group import ActorGroup
    a = train.main(_cfg(tmp_path / "a", **{"training.no_checkpoint": "true"}))
    b = train.main(_cfg(tmp_path / "b", **{"training.no_checkpoint": "true", "training.collocate": "false"}))
    assert len(b["losses"]) == len(a["losses"]) == 3
    for x, y in zip(a["losses"], b["losses"]):
        assert abs(x - y) < 1e-6 * abs(x), (a["losses"], b["losses"])
    g1 = ActorGroup({"tag": "vision", "runtime": "builtin"}, Echo, 2, backend="gloo")
    g2 = ActorGroup({"tag": "text", "runtime": "builtin"}, Echo, 2, collocate=False, backend="gloo", gpu_offset=2)
    try:
        p1, p2 = g1.execute_all("whoami"), g2.execute_all("whoami")
        assert not {x["pid"] for x in p1} & {x["pid"] for x in p2}
    finally:
        g1.shutdown()
        g2.shutdown()


def test_driver_with_accumulation_logging_interval_and_profile_times(tmp_path):
    """Losses are read at logging points only: with ``log_interval=2``, gradient accumulation and ``profile_time``
    the driver still returns one loss per optimizer step, equal to a run that logs every step."""
    from multimodal_training_b200 import train
    base = {"training.no_checkpoint": "true", "training.num_iterations": 5}
    every = train.main(_cfg(tmp_path / "a", **base))
    sparse = train.main(_cfg(tmp_path / "b", **dict(base, **{"training.log_interval": 2, "training.profile_time": "true"})))
    assert len(every["losses"]) == len(sparse["losses"]) == 5
    for a, b in zip(every["losses"], sparse["losses"]):
        assert abs(a - b) < 1e-6 * abs(a)
    acc = train.main(_cfg(tmp_path / "c", **{"training.no_checkpoint": "true", "training.log_interval": 2,
                                              "training.gradient_accumulation_steps": 2}))
    assert acc["steps"] == 3 and len(acc["losses"]) == 3 and acc["losses"][-1] < acc["losses"][0]
