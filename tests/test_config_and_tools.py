"""Config loader / CLI overrides / schema validation, checkpoint split+merge tools, LR schedule, grad-norm
aggregation, vision token calculator, sweep generator."""
import json
import math
import os

import pytest
import torch

from multimodal_training_b200.cli import compute_vision_tokens, merge_checkpoint, split_checkpoint
from multimodal_training_b200.config.loader import ConfigError, load_config, parse_cli, trainer_configs
from multimodal_training_b200.config.model_configs import VLConfig, get_model_config
from multimodal_training_b200.parallel.zero import lr_at

pytestmark = pytest.mark.cpu_only
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_sample_yaml_loads_through_the_hydra_style_cli():
    cfg, ns = parse_cli(["--config-path", os.path.join(ROOT, "configs"), "--config-name", "sample",
                         "training.batch_size=2", "text.parallelism=autotp", "+data.synthetic.image_size=448"])
    assert cfg["training"]["batch_size"] == 2 and cfg["text"]["parallelism"] == "autotp"
    assert cfg["data"]["synthetic"] == {"image_size": 448}
    v, t = trainer_configs(cfg)
    assert v["sequence_parallel_size"] == 8 and t["autotp_size"] == 8 and v["mesh_sp"] == 8 and t["mesh_tp"] == 8
    assert v["learning_rate"] == 5e-5 and "reduce_bucket_size" in v and v["datasets"] == ["laion_pop_train"]


@pytest.mark.parametrize("ov", ["vision.parallelism=ring", "text.dtype=int8", "training.batch_size=0",
                                "training.gradient_accumulation_steps=0", "vision.model_type=llava",
                                "nosuch.key=1", "justakey"])
def test_invalid_configs_are_rejected(ov):
    with pytest.raises(ConfigError):
        load_config(None, [ov])


def test_embedded_model_configs():
    c7, c32 = get_model_config("Qwen/Qwen2.5-VL-7B-Instruct"), get_model_config("qwen2_5_vl_32b")
    assert (c7.text.hidden_size, c7.text.num_hidden_layers, c7.text.num_key_value_heads) == (3584, 28, 4)
    assert (c32.text.hidden_size, c32.text.num_hidden_layers, c32.vision.out_hidden_size) == (5120, 64, 5120)
    assert c7.vision.fullatt_block_indexes == [7, 15, 23, 31] and c7.vision.head_dim == 80
    assert c7.vision.padded_intermediate_size % 8 == 0
    rt = VLConfig.from_dict(json.loads(json.dumps(c7.to_dict())))
    assert rt.text == c7.text and rt.vision == c7.vision
    with pytest.raises(KeyError):
        get_model_config("no-such-model")


def test_lr_schedule_matches_warmup_then_cosine():
    kw = dict(base_lr=1.0, total_steps=100, warmup_steps=10)
    assert lr_at(0, **kw) == 0 and lr_at(5, **kw) == 0.5 and lr_at(10, **kw) == 1.0
    assert abs(lr_at(55, **kw) - 0.5) < 1e-9 and lr_at(100, **kw) < 1e-9
    assert lr_at(50, kind="linear", **kw) == pytest.approx(1 - 40 / 90)
    assert lr_at(50, kind="constant", **kw) == 1.0


def test_aggregate_grad_norms():
    from multimodal_training_b200.train import aggregate_grad_norms
    v = [{"type": "sequence", "sharded": 1.0, "replicated": 0.0}, {"type": "sequence", "sharded": 3.0}]
    t = [{"type": "tensor", "sharded": 2.0, "replicated": 4.0, "tp_size": 2},
         {"type": "tensor", "sharded": 2.0, "replicated": 4.0, "tp_size": 2}]
    assert aggregate_grad_norms(v, t) == pytest.approx(math.sqrt(1 + 3 + 2 + 2 + 4))


def _fake_text_sd(H=8, I=12, V=16, L=2):
    g = torch.Generator().manual_seed(0)
    sd = {"embed_tokens.weight": torch.randn(V, H, generator=g), "norm.weight": torch.ones(H),
          "lm_head.weight": torch.randn(V, H, generator=g)}
    for i in range(L):
        p = f"layers.{i}."
        for n, shape in [("self_attn.q_proj.weight", (H, H)), ("self_attn.k_proj.weight", (H // 2, H)),
                         ("self_attn.v_proj.weight", (H // 2, H)), ("self_attn.o_proj.weight", (H, H)),
                         ("mlp.gate_proj.weight", (I, H)), ("mlp.up_proj.weight", (I, H)),
                         ("mlp.down_proj.weight", (H, I)), ("self_attn.q_proj.bias", (H,)),
                         ("self_attn.k_proj.bias", (H // 2,)), ("self_attn.v_proj.bias", (H // 2,))]:
            sd[p + n] = torch.randn(*shape, generator=g)
        sd[p + "input_layernorm.weight"] = torch.ones(H)
        sd[p + "post_attention_layernorm.weight"] = torch.ones(H)
    return sd


def _shard(sd, tp, r):
    out = {}
    for k, v in sd.items():
        if any(s in k for s in ("o_proj.weight", "down_proj.weight")):
            out[k] = v.chunk(tp, dim=1)[r].clone()
        elif "layernorm" in k or k == "norm.weight":
            out[k] = v.clone()
        else:
            out[k] = v.chunk(tp, dim=0)[r].clone()
    return out


@pytest.mark.parametrize("names", ["{n}_proj", "{n}"])
def test_split_train_merge_round_trip(tmp_path, names):
    """Vision keys as the reference's module tree names them (attn.q_proj, modeling_qwen2_5_vl.py:334-338) and
    as earlier checkpoints of this package did (attn.q)."""
    text = _fake_text_sd()
    vision = {"patch_embed.proj.weight": torch.randn(4, 3, 2, 2, 2), "merger.ln_q.weight": torch.ones(4)}
    for n in "qkv":
        vision[f"blocks.0.attn.{names.format(n=n)}.weight"] = torch.randn(4, 4)
        vision[f"blocks.0.attn.{names.format(n=n)}.bias"] = torch.randn(4)
    full = {**{"model.visual." + k: v for k, v in vision.items()},
            **{"model.language_model." + k: v for k, v in text.items() if not k.startswith("lm_head")},
            "lm_head.weight": text["lm_head.weight"]}
    src = tmp_path / "full.pt"
    torch.save(full, src)
    split_dir = split_checkpoint.split_checkpoint(str(src), str(tmp_path / "split"))
    vs = torch.load(os.path.join(split_dir, "vision_model.pt"))["model"]
    ts = torch.load(os.path.join(split_dir, "text_model.pt"))["model"]
    assert set(vs) == set(vision) and set(ts) == set(text)
    assert os.path.exists(os.path.join(split_dir, "split_metadata.json"))
    # "training" with tp=2: save per-rank shards in the epoch layout, then merge
    ck = tmp_path / "ckpt" / "epoch_0"
    for r in range(2):
        os.makedirs(ck / "vision", exist_ok=True)
        os.makedirs(ck / "text", exist_ok=True)
        torch.save({"model": vs}, ck / "vision" / f"rank_{r}.pt")
        torch.save({"model": _shard(ts, 2, r)}, ck / "text" / f"rank_{r}.pt")
    out = merge_checkpoint.merge_checkpoint(str(ck), str(tmp_path / "merged"), "tiny", 2)
    merged = torch.load(os.path.join(out, "pytorch_model.bin"))
    for k, v in text.items():
        key = k if k.startswith("lm_head") else "language_model." + k
        assert torch.equal(merged[key], v), k
    qkv = torch.cat([vision[f"blocks.0.attn.{names.format(n=n)}.weight"] for n in "qkv"])
    assert torch.equal(merged["visual.blocks.0.attn.qkv.weight"], qkv)      # re-fused for stock HF
    assert not any(".attn.q" in k and ".attn.qkv" not in k for k in merged)
    assert json.load(open(os.path.join(out, "merge_metadata.json")))["vision_qkv"] == "fused"


def test_vision_token_calculator_and_sweep_generator(tmp_path, capsys):
    assert compute_vision_tokens.vision_tokens(896)["patches"] == 4096
    assert compute_vision_tokens.vision_tokens(3584)["merged_tokens"] == 16384
    assert compute_vision_tokens.main([]) == 0 and "65536" in capsys.readouterr().out
    import importlib.util
    spec = importlib.util.spec_from_file_location("gen", os.path.join(ROOT, "experiments", "generate_configs.py"))
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    assert gen.main(["--output-dir", str(tmp_path / "sweep"), "--synthetic"]) == 0
    names = (tmp_path / "sweep" / "manifest.txt").read_text().split()
    assert len(names) == 2 * 6 * 2 * 4
    cfg = load_config(tmp_path / "sweep" / "configs" / (names[0] + ".yaml"))
    assert cfg["data"]["force_fixed_size"] and cfg["data"]["synthetic"]["image_size"] == 448
    big = load_config(tmp_path / "sweep" / "configs" / "32b_64k_tokens_sequence_bs2.yaml")
    assert big["deepspeed"]["reduce_bucket_size"] == 100000000 and big["training"]["parallel_size"] == 8
    runner = (tmp_path / "sweep" / "run_sweep.sh").read_text()
    assert "python -m multimodal_training_b200.train --config-path" in runner and "__LAUNCH__" not in runner
    assert 'HERE="$PWD"' in runner and '--config-path "$HERE/configs"' in runner   # $PWD changes with the cd to the repo
    assert gen.main(["--output-dir", str(tmp_path / "sweep2"), "--synthetic", "--launcher", "torchrun"]) == 0
    runner = (tmp_path / "sweep2" / "run_sweep.sh").read_text()
    assert "--nproc-per-node" in runner and "-m multimodal_training_b200.train_spmd --config-path" in runner
    # the rank count comes from the config itself: check the embedded one-liner on a generated file
    import subprocess
    import sys
    name = "7b_1k_tokens_sequence_bs1"
    code = ("import yaml; t = yaml.safe_load(open('%s'))['training']; print(t['parallel_size'] * t.get('dp_size', 1))"
            % (tmp_path / "sweep2" / "configs" / (name + ".yaml")))
    assert "import yaml; t = yaml.safe_load(open('$HERE/configs/$name.yaml'))['training']" in runner
    assert subprocess.run([sys.executable, "-c", code], capture_output=True, text=True).stdout.strip() == "4"
    assert subprocess.run(["bash", "-n", str(tmp_path / "sweep2" / "run_sweep.sh")]).returncode == 0


def test_phase_timer_and_chrome_trace(tmp_path):
    import json
    import time
    from multimodal_training_b200.utils import tracing
    t = tracing.PhaseTimer(use_cuda=False)
    for _ in range(2):
        with t.phase("a"):
            time.sleep(0.002)
        with t.phase("b"):
            pass
        t.end_step()
    s = t.summary()
    assert set(s) == {"a", "b"} and s["a"] >= 1.0 and s["b"] < s["a"]
    path = t.chrome_trace(str(tmp_path / "trace.json"), rank=3)
    ev = json.load(open(path))["traceEvents"]
    assert len(ev) == 4 and ev[0]["pid"] == 3 and ev[0]["args"]["step"] == 0 and ev[-1]["args"]["step"] == 1
    with tracing.trace_range("noop"):        # off by default: must be a plain no-op
        pass


def test_checkpoint_policy_decision():
    from multimodal_training_b200.utils.checkpointing import decide
    assert decide(True, 0) is True and decide(False, 10 ** 15) is False
    assert decide("false", 1) is False and decide("true", 1) is True
    assert decide("auto", 10 ** 15, "cpu") is False          # no device memory to protect on the CPU path


def test_staging_ring_reuses_a_buffer_only_after_its_copy_finished():
    from multimodal_training_b200.trainers.context import StagingRing
    ring = StagingRing(slots=3, pin=False)
    a = ring.acquire(4, 8, torch.float32)
    b = ring.acquire(4, 8, torch.float32)
    c = ring.acquire(6, 8, torch.float32)
    assert a.shape == (4, 8) and c.shape == (6, 8)
    assert len({a.data_ptr(), b.data_ptr(), c.data_ptr()}) == 3        # three steps in flight never share memory

    class Event:
        waited = 0

        def synchronize(self):
            Event.waited += 1

    ring.slots[0][1] = Event()               # as recorded behind the copy out of the first buffer
    again = ring.acquire(3, 8, torch.float32)
    assert again.data_ptr() == a.data_ptr() and again.shape == (3, 8) and Event.waited == 1
    assert ring.slots[0][1] is None
    bigger = ring.acquire(16, 8, torch.float32)                           # second slot grows
    assert bigger.shape == (16, 8) and bigger.data_ptr() != b.data_ptr()
    ring.copied()                                                         # no events without pinned memory
    assert ring.slots[1][1] is None


def test_token_buckets_bound_the_number_of_checkpointing_decisions():
    from multimodal_training_b200.utils.checkpointing import bucket_tokens
    assert [bucket_tokens(n) for n in (1, 1024, 1025, 1040, 2048, 2049, 4096, 36864)] == \
        [1024, 1024, 1280, 1280, 2048, 2560, 4096, 40960]
    sizes = {bucket_tokens(n) for n in range(1000, 70000, 7)}
    assert len(sizes) <= 4 * 7 + 1 and all(bucket_tokens(n) >= n for n in range(1, 70000, 97))


def test_fused_comm_auto_is_on_for_data_sets_too():
    """Heap regions are sized per step and grow, so ``auto`` no longer depends on the batches having one shape."""
    from multimodal_training_b200.trainers.trainer import Trainer
    want = lambda cfg: Trainer(cfg)._want_fused_comm()  # noqa: E731
    assert want({"synthetic": {"image_size": 448}}) and want({})
    assert want({"fused_comm": "auto", "synthetic": {"image_size": 448}}) and want({"fused_comm": "auto"})
    assert want({"fused_comm": True}) and want({"fused_comm": "true"})
    assert not want({"fused_comm": False, "synthetic": {"image_size": 448}}) and not want({"fused_comm": "false"})
    v, _ = trainer_configs(load_config(None, []))
    assert v["fused_comm"] == "auto"


def test_zero_stage_three_is_rejected_only_where_it_would_be_used():
    """``zero_stage`` is consulted with ``parallelism: deepspeed`` only (as in the reference): stages 0-2 run as the
    flat-buffer ZeRO optimizer, stage 3 (parameter partitioning) is refused instead of being mapped silently."""
    load_config(None, ["text.parallelism=tensor", "text.zero_stage=3"])           # ignored in this mode
    load_config(None, ["text.parallelism=deepspeed", "text.zero_stage=2"])
    with pytest.raises(ConfigError, match="zero_stage"):
        load_config(None, ["text.parallelism=deepspeed", "text.zero_stage=3"])
    with pytest.raises(ConfigError, match="zero_stage"):
        load_config(None, ["vision.parallelism=deepspeed", "vision.zero_stage=3"])


def test_idle_gap_summary_merges_streams_and_sets_the_startup_gap_aside():
    from multimodal_training_b200.utils.idle_gaps import merge_intervals, short_name, summarize
    assert merge_intervals([(5, 9), (0, 3), (2, 4), (9, 10)]) == [(0, 4), (5, 10)]
    # two streams overlapping, a 5 ms hole right after the first kernel (empty launch queue at trace start), then
    # 2000 kernels of 18 us every 20 us
    iv = [(0, 10), (5000, 5010)] + [(5010 + i * 20, 5010 + i * 20 + 18) for i in range(2000)] + [(6000, 6015)]
    out = summarize(iv, steps=2)
    assert abs(out["startup_gap_ms"] - 4.99) < 1e-6
    assert abs(out["idle_ms_per_step"] - 2.0) < 0.01 and abs(out["idle_share"] - 0.1) < 0.002
    assert short_name("void (anonymous namespace)::gemm_bf16_tcgen05<256, 2>(CUtensorMap_st, int)") == "gemm_bf16_tcgen05"
