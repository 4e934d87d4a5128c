"""Config composition, validation, batch scaling, LR schedule, precision policy, logger, monitoring (CPU only)."""

import json
import math
from pathlib import Path

import pytest
import torch

from mini_train_sys_b200.models import ModelConfig
from mini_train_sys_b200.runtime import config as cfgmod
from mini_train_sys_b200.runtime.logger import (JsonlLogger, balance_heatmap, build_event_logger, encode_png_rgb,
                                                format_console_event)
from mini_train_sys_b200.runtime.monitoring import (GpuUtilizationMonitor, distributed_gpu_utilization, distributed_mean,
                                                    distributed_mean_tensors)
from mini_train_sys_b200.runtime.scaling import resolve_batch_scale
from mini_train_sys_b200.train.lr_scheduler import LearningRateScheduler, lr_scale, resolve_total_steps
from mini_train_sys_b200.train.precision import resolve_precision_policy

ROOT = Path(__file__).resolve().parents[1]


def test_every_shipped_run_and_model_yaml_loads():
    models = runs = 0
    for path in sorted((ROOT / "configs").rglob("*.yaml")):
        payload = cfgmod.load_yaml_dict(path)      # every file, fragments included, must parse and resolve `extends`
        if set(payload) == {"model"}:
            ModelConfig(**payload["model"])
            models += 1
        elif path.parent.name == "runs" or path.name.startswith("train_") or path.name.endswith("_pretrain.yaml"):
            payload.pop("model", None)
            cfg = cfgmod.experiment_config_from_dict(payload)   # complete run files validate as a whole
            assert cfg.parallel.strategy in ("single", "ddp", "fsdp", "ep")
            runs += 1
    assert models >= 7 and runs >= 10


def test_extends_merges_in_order_and_detects_cycles(tmp_path):
    (tmp_path / "base.yaml").write_text("train:\n  batch_size: 4\n  log_interval: 7\noptimizer:\n  lr: 0.1\n")
    (tmp_path / "mid.yaml").write_text("extends: base.yaml\ntrain:\n  batch_size: 8\n")
    (tmp_path / "top.yaml").write_text("extends: [mid.yaml]\noptimizer:\n  lr: 0.5\n")
    merged = cfgmod.load_yaml_dict(tmp_path / "top.yaml")
    assert merged == {"train": {"batch_size": 8, "log_interval": 7}, "optimizer": {"lr": 0.5}}
    (tmp_path / "a.yaml").write_text("extends: b.yaml\n")
    (tmp_path / "b.yaml").write_text("extends: a.yaml\n")
    with pytest.raises(ValueError, match="cycle"):
        cfgmod.load_yaml_dict(tmp_path / "a.yaml")


@pytest.mark.parametrize("section,kwargs", [
    (cfgmod.BackendConfig, {"ops": "jax"}), (cfgmod.ParallelConfig, {"strategy": "pp"}),
    (cfgmod.FSDPConfig, {"sharding_strategy": "no_shard"}), (cfgmod.TrainConfig, {"max_steps": None, "epochs": None}),
    (cfgmod.TrainConfig, {"batch_size_scaling": "linear"}), (cfgmod.CheckpointConfig, {"keep_safety": 1}),
    (cfgmod.DataConfig, {"source": "tokens"}), (cfgmod.DataConfig, {"packing": "randomized_documents"}),
    (cfgmod.LRSchedulerConfig, {"decay_steps": 10, "warmup_steps": 20}), (cfgmod.OptimizerConfig, {"name": "sgd"}),
    (cfgmod.CommConfig, {"engine": "mpi"}), (cfgmod.DataConfig, {"num_workers": 0, "persistent_workers": True}),
])
def test_invalid_sections_are_rejected(section, kwargs):
    with pytest.raises(ValueError):
        section(**kwargs)


def test_reference_backend_names_stay_valid_and_new_sections_default():
    cfg = cfgmod.experiment_config_from_dict({"backend": {"ops": "triton"}, "parallel": {"strategy": "fsdp"}})
    assert cfg.backend.ops == "triton" and cfg.parallel.comm.engine == "auto" and cfg.parallel.ep.capacity_factor is None


def test_model_config_validation_and_counts():
    with pytest.raises(ValueError):
        ModelConfig(hidden_size=100, n_heads=12)
    with pytest.raises(ValueError):
        ModelConfig(ffn_type="moe", experts_per_token=9, num_experts=8)
    payload = cfgmod.load_yaml_dict(ROOT / "configs" / "synbios_moe" / "model.yaml")["model"]
    assert ModelConfig(**payload).param_count() == 293_494_272
    dense = cfgmod.load_yaml_dict(ROOT / "configs" / "model_125m_dense.yaml")["model"]
    assert ModelConfig(**dense).param_count() == 162_417_408


def test_linear_batch_scaling():
    train = cfgmod.TrainConfig(batch_size=24, reference_global_batch_size=96, batch_size_scaling="linear")
    out = resolve_batch_scale(train, cfgmod.OptimizerConfig(lr=1e-3), cfgmod.LRSchedulerConfig(warmup_steps=1000, decay_steps=5000),
                              world_size=8)
    assert out.scale == 2.0 and out.optimizer.lr == pytest.approx(2e-3)
    assert out.lr_scheduler.warmup_steps == 500 and out.lr_scheduler.decay_steps == 2500
    none = resolve_batch_scale(cfgmod.TrainConfig(batch_size=24), cfgmod.OptimizerConfig(), cfgmod.LRSchedulerConfig(), world_size=8)
    assert none.scale == 1.0 and none.global_batch_size == 192


def test_lr_schedule_shape_and_state():
    cfg = cfgmod.LRSchedulerConfig(schedule="cosine", warmup_steps=10, min_lr_ratio=0.1)
    assert lr_scale(cfg, 0, 100) == pytest.approx(0.1)
    assert lr_scale(cfg, 9, 100) == pytest.approx(1.0)
    assert lr_scale(cfg, 10, 100) == pytest.approx(1.0)
    assert lr_scale(cfg, 55, 100) == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.5)))
    assert lr_scale(cfg, 1000, 100) == pytest.approx(0.1)
    assert lr_scale(cfgmod.LRSchedulerConfig(schedule="constant", warmup_steps=0), 5, 10) == 1.0
    assert resolve_total_steps(max_steps=50, epochs=2, steps_per_epoch=10) == 20
    with pytest.raises(ValueError):
        resolve_total_steps(max_steps=None, epochs=None, steps_per_epoch=10)
    opt = torch.optim.SGD([torch.zeros(1, requires_grad=True)], lr=2.0)
    sched = LearningRateScheduler(opt, cfg, total_steps=100)
    sched.step(9)
    assert opt.param_groups[0]["lr"] == pytest.approx(2.0)
    other = LearningRateScheduler(torch.optim.SGD([torch.zeros(1, requires_grad=True)], lr=2.0), cfg, total_steps=100)
    other.load_state_dict(sched.state_dict())
    assert other.get_last_lr() == sched.get_last_lr()


def test_precision_policy_on_cpu():
    pol = resolve_precision_policy("auto", torch.device("cpu"))
    assert pol.name == "fp32" and not pol.autocast_enabled and not pol.grad_scaling_enabled
    with pytest.raises(ValueError):
        resolve_precision_policy("fp16", torch.device("cpu"))
    with pytest.raises(ValueError):
        resolve_precision_policy("fp8", torch.device("cpu"))


def test_console_formatting_and_jsonl_sink(tmp_path):
    line = format_console_event({"event": "train", "batch": 3, "batches_total": 10, "loss": 1.23456, "lr": 3e-4, "grad_norm": 0.5,
                                 "tokens_per_sec": 1234.5, "progress_percent": 30.0, "eta_seconds": 3700})
    assert line.startswith("[train] batch 3/10") and "loss 1.23456" in line and "ETA 1:01:40" in line
    assert format_console_event({"event": "init", "run": "r", "device": "cpu", "parallel": "single", "world_size": 1, "params": 5}) \
        == "[init] run=r device=cpu strategy=single world=1 params=5"
    sink = JsonlLogger(tmp_path / "a" / "events.jsonl")
    sink.log_event({"event": "x", "step": 1, "v": [1, 2]})
    sink.close()
    sink.close()
    sink.log_event({"event": "ignored"})
    assert json.loads((tmp_path / "a" / "events.jsonl").read_text().strip()) == {"event": "x", "step": 1, "v": [1, 2]}


def test_png_encoder_and_balance_heatmap():
    img = balance_heatmap(torch.tensor([[0.0, 0.125, 0.25], [0.125, 0.125, 0.125]]))
    assert img.shape == (3, 2, 3) and float(img.min()) >= 0 and float(img.max()) <= 1
    png = encode_png_rgb((img * 255).round().to(torch.uint8).permute(1, 2, 0).contiguous())
    assert png[:8] == b"\x89PNG\r\n\x1a\n" and png[12:16] == b"IHDR" and png[-8:-4] == b"IEND"


def test_logger_stack_respects_rank(monkeypatch, tmp_path):
    monkeypatch.setenv("RANK", "1")
    logger = build_event_logger(cfgmod.LoggingConfig(tensorboard=False, log_dir=str(tmp_path)), run_name="r")
    assert type(logger).__name__ == "NullLogger"
    monkeypatch.setenv("RANK", "0")
    logger = build_event_logger(cfgmod.LoggingConfig(console=False, tensorboard=False, log_dir=str(tmp_path)), run_name="r")
    logger.log_event({"event": "train", "step": 1})
    logger.close()
    assert len(list(tmp_path.rglob("events.jsonl"))) == 1


class _FakeNvml:
    class _Rates:
        gpu, memory = 73.0, 41.0

    def __init__(self):
        self.shutdowns = 0

    def nvmlInit(self):
        pass

    def nvmlDeviceGetCount(self):
        return 2

    def nvmlDeviceGetHandleByIndex(self, i):
        return i

    def nvmlDeviceGetUUID(self, h):
        return [b"GPU-aaaa-1111", b"GPU-bbbb-2222"][h]

    def nvmlDeviceGetUtilizationRates(self, h):
        return self._Rates()

    def nvmlShutdown(self):
        self.shutdowns += 1


def test_gpu_monitor_against_a_fake_nvml():
    fake = _FakeNvml()
    mon = GpuUtilizationMonitor(torch.device("cpu"), sample_interval_seconds=0.01, nvml=fake, device_uuid="GPU-BBBB-2222")
    mon.start()
    assert mon.available
    import time

    time.sleep(0.05)
    stats = mon.read_interval()
    mon.close()
    assert stats["gpu_compute_utilization_percent_local_mean"] == 73.0 and stats["gpu_utilization_samples_local"] >= 2
    assert fake.shutdowns == 1
    merged = distributed_gpu_utilization(stats, torch.device("cpu"))
    assert merged["gpu_utilization_available"] == 1 and merged["gpu_memory_controller_utilization_percent_max"] == 41.0
    assert distributed_gpu_utilization({}, torch.device("cpu")) == {"gpu_utilization_available": 0}


def test_single_process_reductions_are_identity():
    assert distributed_mean({"b": 2.0, "a": 1.0}, torch.device("cpu")) == {"a": 1.0, "b": 2.0}
    out = distributed_mean_tensors({"m": torch.arange(6.0).view(2, 3)}, torch.device("cpu"))
    assert out == {"m": [[0.0, 1.0, 2.0], [3.0, 4.0, 5.0]]}


def test_build_config_profiles_and_cache_key():
    from mini_train_sys_b200.ops.build import NVCC_FLAGS, BuildConfig

    assert "arch=compute_100a,code=sm_100a" in NVCC_FLAGS and "-lineinfo" in NVCC_FLAGS
    release = BuildConfig.from_env({})
    traced = BuildConfig.from_env({"MTS_BUILD_PROFILE": "trace-attention", "MTS_EXTRA_NVCC_FLAGS": "-DFOO=1"})
    assert release.profile == "release" and "-DMTS_ATTN_TRACE" in traced.nvcc_flags() and "-DFOO=1" in traced.nvcc_flags()
    assert release.cache_key() != traced.cache_key() and release.cache_key() == BuildConfig().cache_key()
    with pytest.raises(ValueError):
        BuildConfig.from_env({"MTS_BUILD_PROFILE": "nope"})


def test_bounds_checking_profile_compiles_the_kernels_that_use_it(tmp_path):
    """The ``debug-bounds`` build profile: every source that uses the checked accessor must still compile with it on."""

    import shutil
    import subprocess

    from mini_train_sys_b200.ops.build import CSRC, PROFILES, BuildConfig

    assert "-DMTS_DEBUG_BOUNDS" in PROFILES["debug-bounds"]
    assert "-DMTS_DEBUG_BOUNDS" in BuildConfig(profile="debug-bounds").nvcc_flags()
    assert BuildConfig(profile="debug-bounds").cache_key() != BuildConfig().cache_key()
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not shutil.which(nvcc):
        pytest.skip("nvcc not available")
    users = [p for p in sorted(CSRC.glob("*.cu")) if "MTS_IN_BOUNDS" in p.read_text()]
    assert {p.name for p in users} >= {"embedding.cu", "router_moe.cu", "comm.cu"}
    for src in users[:2]:     # two translation units are enough to catch a broken header; each takes a few seconds
        done = subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "--expt-relaxed-constexpr",
                               "-DMTS_DEBUG_BOUNDS", "-I", str(CSRC), "-c", str(src), "-o", str(tmp_path / (src.stem + ".o"))],
                              capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]


# ---- memory plan --------------------------------------------------------------------------------------------------------
def _model_from(path: str) -> ModelConfig:
    import yaml

    return ModelConfig(**yaml.safe_load((ROOT / path).read_text())["model"])


def test_memory_plan_static_part_equals_the_engine_buffers():
    """The resident part of the plan against a real engine: every buffer the flat engine allocates for a model, summed."""

    from mini_train_sys_b200.models import MiniTransformer, get_ops_backend
    from mini_train_sys_b200.parallel.flat_engine import FlatDataParallel
    from mini_train_sys_b200.runtime.memory_plan import plan_memory

    for kind in ("dense", "moe"):
        cfg = ModelConfig(vocab_size=1000, seq_len=32, n_layers=3, n_heads=4, hidden_size=128, intermediate_size=256, ffn_type=kind,
                          num_experts=4, experts_per_token=2, tie_word_embeddings=(kind == "moe"))
        torch.manual_seed(0)
        engine = FlatDataParallel(MiniTransformer(cfg, get_ops_backend("torch")), mode="shard")
        held = 0
        for unit in engine.units:
            tensors = [unit.master, unit.exp_avg, unit.exp_avg_sq, unit.grad_shard, unit.grad_full.tensor, unit.low_shard.tensor]
            if unit.gathered is not None:
                tensors.append(unit.gathered.tensor)
            held += sum(t.numel() * t.element_size() for t in tensors)
        # on a CPU the engine keeps its "low precision" buffers in fp32: plan with 4-byte weights
        plan = plan_memory(cfg, strategy="single", low_bytes=4)
        assert plan.static_bytes() == 28 * cfg.param_count()                       # 16 + 4 + 4 + 4 bytes per parameter
        padding = len(engine.units) * 64 * 28                                      # units are padded to a multiple of 64 elements
        assert plan.static_bytes() <= held <= plan.static_bytes() + padding, (kind, held, plan.static_bytes())


def test_memory_plan_reproduces_the_measured_peaks():
    """``max_memory_allocated`` (GiB) of benchmark runs of this repository on B200: model, strategy, ranks, sharding, local batch."""

    from mini_train_sys_b200.runtime.memory_plan import GIB, plan_memory

    moe293, dense125, moe125 = (_model_from(p) for p in ("configs/synbios_moe/model.yaml", "configs/model_125m_dense.yaml",
                                                         "configs/model_125m_moe.yaml"))
    measured = [
        (moe293, "single", 1, "full_shard", 96, 30.51), (moe293, "single", 1, "full_shard", 24, 12.88),
        (moe293, "fsdp", 2, "full_shard", 96, 26.23), (moe293, "fsdp", 2, "full_shard", 24, 8.61), (moe293, "fsdp", 2, "shard_grad_op", 96, 26.08),
        (moe293, "fsdp", 4, "full_shard", 96, 25.14), (moe293, "fsdp", 4, "full_shard", 24, 7.52),
        (moe293, "fsdp", 8, "full_shard", 96, 24.59), (moe293, "fsdp", 8, "full_shard", 24, 6.96),
        (dense125, "ddp", 2, "full_shard", 32, 15.82), (dense125, "ddp", 4, "full_shard", 32, 15.20), (dense125, "ddp", 8, "full_shard", 32, 14.91),
        (moe125, "fsdp", 2, "full_shard", 16, 13.95), (moe125, "fsdp", 4, "full_shard", 16, 12.22),
        (moe125, "ep", 2, "full_shard", 16, 21.63), (moe125, "ep", 4, "full_shard", 16, 18.82),
    ]
    for model, strategy, world, sharding, batch, gib in measured:
        plan = plan_memory(model, strategy=strategy, world_size=world, sharding=sharding, local_batch_hint=batch)
        predicted = plan.total_bytes(batch, allocator_only=True) / GIB
        assert predicted == pytest.approx(gib, rel=0.02), (strategy, world, sharding, batch, predicted, gib)
        # what the allocator does not see: nothing on one rank, the symmetric buffers otherwise
        hidden = plan.total_bytes(batch) - plan.total_bytes(batch, allocator_only=True)
        assert (hidden == 0) == (world == 1) and hidden <= 7 * model.param_count() + plan.static.get("expert_exchange_regions", 0)


def test_memory_plan_orderings_limits_and_cli(tmp_path):
    import subprocess
    import sys

    from mini_train_sys_b200.runtime.memory_plan import GIB, plan_memory

    model = _model_from("configs/synbios_moe/model.yaml")
    full, grad_op = (plan_memory(model, strategy="fsdp", world_size=8, sharding=s) for s in ("full_shard", "shard_grad_op"))
    assert full.static_bytes() < grad_op.static_bytes() < plan_memory(model).static_bytes()
    assert plan_memory(model, activation_checkpointing=True).activation_bytes(1) < 0.5 * plan_memory(model).activation_bytes(1)
    best = full.max_local_batch(180 * GIB)
    assert 500 < best < 800 and full.total_bytes(best) <= 0.9 * 180 * GIB < full.total_bytes(best + 1)
    assert full.max_local_batch(1 * GIB) == 0
    # a model whose full-size fp32 gradient buffer alone exceeds the device: the plan says so instead of returning a batch
    huge = ModelConfig(vocab_size=128000, seq_len=4096, n_layers=80, n_heads=64, hidden_size=8192, intermediate_size=28672)
    plan = plan_memory(huge, strategy="fsdp", world_size=8)
    assert plan.max_local_batch(180 * GIB) == 0 and any("gradient buffer" in n for n in plan.notes)
    with pytest.raises(ValueError):
        plan_memory(model, strategy="ep", world_size=3)
    with pytest.raises(ValueError):
        plan_memory(_model_from("configs/model_125m_dense.yaml"), strategy="ep", world_size=2)
    done = subprocess.run([sys.executable, str(ROOT / "scripts" / "plan_memory.py"), "--config",
                           str(ROOT / "configs" / "server" / "b200_180gb" / "runs" / "fsdp_8gpu.yaml"), "--model-config",
                           str(ROOT / "configs" / "synbios_moe" / "model.yaml")], capture_output=True, text=True, timeout=120)
    report = json.loads(done.stdout)
    assert done.returncode == 0 and report["fits"] and report["world_size"] == 8 and report["local_batch"] == 96
    assert report["max_memory_allocated_gib"] == pytest.approx(24.59, rel=0.03) and report["max_local_batch"] == best
    tight = subprocess.run([sys.executable, str(ROOT / "scripts" / "plan_memory.py"), "--model-config", str(ROOT / "configs" / "synbios_moe" / "model.yaml"),
                            "--local-batch", "96", "--device-gb", "24"], capture_output=True, text=True, timeout=120)
    assert tight.returncode == 1 and not json.loads(tight.stdout)["fits"]


# ---- server preflight -----------------------------------------------------------------------------------------------------
def test_server_check_reports_errors_on_a_machine_without_gpus_and_reads_nvlink_listings():
    from mini_train_sys_b200.runtime.server_check import collect_server_status, nvlink_findings, parse_nvlink_status

    listing = "\n".join(["GPU 0: NVIDIA B200 (UUID: GPU-00000000-0000-0000-0000-000000000000)",
                         *[f"\t Link {k}: 53.125 GB/s" for k in range(18)],
                         "GPU 1: NVIDIA B200 (UUID: GPU-11111111-1111-1111-1111-111111111111)",
                         *[f"\t Link {k}: 53.125 GB/s" for k in range(16)], "\t Link 16: <inactive>", "\t Link 17: <inactive>", "unrelated line"])
    status = parse_nvlink_status(listing)
    assert status[0] == {"active_links": 18, "inactive_links": 0, "gbs_per_direction": pytest.approx(956.25)}
    assert status[1]["active_links"] == 16 and status[1]["inactive_links"] == 2
    assert nvlink_findings(status) == ["GPU 1: 16 of 18 NVLink links active (2 reported inactive)"]
    assert parse_nvlink_status("") == {} and nvlink_findings({}) == []
    if not torch.cuda.is_available():
        report = collect_server_status(expected_gpus=1, min_free_disk_gb=0.0, require_nvcc=False)
        assert not report["ok"] and "CUDA is not available" in report["errors"] and report["gpu_count"] == 0 and report["nvlink"] == {}
        assert report["checkout"] is not None and isinstance(report["extension_built"], bool)


# ---- step roofline ----------------------------------------------------------------------------------------------------------
def test_step_roofline_counts_the_model_flops_and_every_pass_once():
    import subprocess
    import sys

    from mini_train_sys_b200.runtime.step_model import step_roofline, step_work

    peaks = {"hbm_gbs": 6553.9, "bf16_tflops": 1650.4, "bf16_tflops_sustained": 1371.8, "source": "test"}
    for path, batch in (("configs/synbios_moe/model.yaml", 96), ("configs/model_125m_dense.yaml", 32), ("configs/model_debug_moe.yaml", 4)):
        model = _model_from(path)
        tokens = batch * model.seq_len
        report = step_roofline(model, batch, peaks=peaks, measured_ms=100.0)
        # the contractions of a step are 6 FLOPs per token and active matrix parameter (router and embedding gather aside)
        matrix = model.active_param_count() - (model.n_layers * model.num_experts * model.hidden_size if model.is_moe else 0)
        gemms = [w for w in step_work(model, batch) if w.kind == "gemm"]
        assert sum(w.count * w.flops for w in gemms) == pytest.approx(6.0 * tokens * matrix, rel=1e-9)
        assert len(gemms) == (6 + 6 + 3) and all(w.flops > 0 and w.bytes == 0 for w in gemms)
        assert sum(report["bound_ms_by_kind"].values()) == pytest.approx(report["bound_ms_sustained"], abs=2e-3)
        assert report["bound_ms_burst"] <= report["bound_ms_sustained"] and report["achieved_fraction_of_sustained_bound"] == pytest.approx(report["bound_ms_sustained"] / 100.0, abs=1e-3)
    headline = step_roofline(_model_from("configs/synbios_moe/model.yaml"), 96, peaks=peaks)
    assert headline["bound_ms_sustained"] == pytest.approx(36.4, abs=0.3) and headline["bound_ms_by_kind"]["gemm"] == pytest.approx(26.6, abs=0.2)
    done = subprocess.run([sys.executable, str(ROOT / "scripts" / "step_roofline.py"), "--model-config", str(ROOT / "configs" / "synbios_moe" / "model.yaml"),
                           "--local-batch", "96", "--measured-ms", "62.69"], capture_output=True, text=True, timeout=120)
    assert done.returncode == 0 and "of the sustained bound" in done.stdout and "| logits | gemm | 1 |" in done.stdout


def test_nvlink_traffic_per_path_matches_the_hand_count():
    from mini_train_sys_b200.runtime.step_model import comm_work

    model = _model_from("configs/synbios_moe/model.yaml")
    grads, weights = 4 * model.param_count(), 2 * model.param_count()
    assert comm_work(model, 96, strategy="single", world_size=1) == [] and comm_work(model, 96, strategy="fsdp", world_size=1) == []
    full = {row["path"].split(",")[0]: row for row in comm_work(model, 96, strategy="fsdp", world_size=8)}
    assert full["gradient reduce-scatter"]["gb_in"] == pytest.approx(7 / 8 * grads / 1e9, rel=1e-3)          # 1.027 GB
    assert full["gradient reduce-scatter"]["alone_ms"] == pytest.approx(1.334, abs=2e-3) and full["gradient reduce-scatter"]["launches"] == 13
    assert full["parameter all-gather into staging slots"]["gb_in"] == pytest.approx(2 * 7 / 8 * weights / 1e9, rel=1e-3)
    resident = {row["path"].split(":")[0].split(",")[0]: row for row in comm_work(model, 96, strategy="fsdp", world_size=8, sharding="shard_grad_op")}
    assert "parameter all-gather into staging slots" not in resident and resident["AdamW"]["gb_out"] == pytest.approx(7 / 8 * weights / 1e9, rel=1e-3)
    switch = comm_work(model, 96, strategy="fsdp", world_size=8, multimem=True)[0]
    assert switch["gb_in"] == pytest.approx(grads / 8 / 1e9, rel=1e-3) and switch["gb_out"] == 0.0
    moe = _model_from("configs/model_125m_moe.yaml")
    ep = comm_work(moe, 16, strategy="ep", world_size=4)
    rows = 16 * moe.seq_len * moe.experts_per_token
    assert ep[-1]["gb_in"] == pytest.approx(2 * moe.n_layers * 0.75 * rows * moe.hidden_size * 2 / 1e9, rel=1e-3) and ep[-1]["launches"] == 2 * moe.n_layers
    experts = moe.n_layers * moe.num_experts * 3 * moe.hidden_size * moe.intermediate_size
    assert ep[0]["gb_in"] == pytest.approx(0.75 * 4 * (moe.param_count() - experts) / 1e9, rel=1e-3)         # expert gradients stay local


def test_memory_plan_event_of_shipped_run_files():
    from mini_train_sys_b200.runtime.memory_plan import GIB, memory_plan_event

    cfg = cfgmod.load_experiment(ROOT / "configs" / "server" / "b200_180gb" / "runs" / "fsdp_8gpu.yaml", ROOT / "configs" / "synbios_moe" / "model.yaml")
    event = memory_plan_event(cfg, world_size=8, device_bytes=180 * GIB)
    assert event["event"] == "memory_plan" and event["fits"] and event["local_batch"] == 96
    assert event["planned_max_memory_allocated_gib"] == pytest.approx(24.59, rel=0.03) and event["max_local_batch"] > 500
    assert not memory_plan_event(cfg, world_size=8, device_bytes=16 * GIB)["fits"]
    json.dumps(event)                                                    # plain values only: it goes straight into the event log
    for path in sorted((ROOT / "configs").rglob("*.yaml")):              # every shipped run file: an event or None, never an exception
        try:
            run = cfgmod.load_experiment(path)
        except Exception:                                                # model files and fragments are not run files
            continue
        for world in (1, 2, 8):
            out = memory_plan_event(run, world_size=world, device_bytes=180 * GIB)
            assert out is None or (out["planned_peak_gib"] > 0 and isinstance(out["fits"], bool))
    debug = cfgmod.load_experiment(ROOT / "configs" / "train_debug.yaml")
    assert memory_plan_event(debug, world_size=1, device_bytes=180 * GIB) is None        # no model section: nothing to plan
