"""Benchmark harness on CPU: parity statistics, operator worker, Nsight command builder, distributed suites over Gloo."""

import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]


def test_close_stats_streams_and_flags_violations():
    from mini_train_sys_b200.bench.measurement import close_stats

    a = torch.linspace(-1, 1, 10_000)
    ok = close_stats(a + 1e-4, a, atol=1e-3, rtol=0.0)
    assert ok["passed"] and ok["max_abs"] == pytest.approx(1e-4, rel=1e-2) and ok["cosine"] > 0.999999
    b = a.clone(); b[17] += 1.0
    bad = close_stats(b, a, atol=1e-3, rtol=0.0)
    assert not bad["passed"] and bad["violations"] == 1
    assert not close_stats(torch.tensor([float("nan")]), torch.tensor([0.0]), atol=1.0, rtol=0.0)["passed"]


@pytest.mark.parametrize("kernel", ["embedding", "rmsnorm", "swiglu", "rope", "attention", "cross_entropy", "fused_linear_cross_entropy", "linear",
                                    "router", "router_logits", "fused_moe"])
def test_operator_cases_agree_between_library_and_oracle_back_ends(kernel):
    from mini_train_sys_b200.bench.measurement import correctness_stats
    from mini_train_sys_b200.bench.operators import OperatorProfile, build_case
    from mini_train_sys_b200.models import get_ops_backend

    prof = OperatorProfile("tiny", hidden=64, intermediate=96, heads=2, head_dim=32, vocab=257, seq_len=16, experts=4, top_k=2)
    case = build_case(kernel, prof, 64)
    with torch.autocast("cpu", dtype=torch.bfloat16):
        stats = correctness_stats(case, get_ops_backend("torch"), get_ops_backend("reference"), torch.device("cpu"),
                                  relative_gate=(2e-2, 0.999))
    assert stats["passed"], stats


def test_bench_ops_worker_cli_runs_on_cpu():
    out = subprocess.run([sys.executable, str(ROOT / "scripts" / "bench_ops.py"), "_worker", "--kernel", "swiglu", "--profile",
                          "project_formal", "--tokens", "512", "--providers", "torch,reference", "--warmup", "1", "--iters", "3"],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    rec = json.loads(out.stdout.strip().splitlines()[-1])
    assert rec["status"] == "ok" and {r["provider"] for r in rec["rows"]} == {"torch", "reference"}
    ref_row = next(r for r in rec["rows"] if r["provider"] == "reference")
    assert ref_row["correctness"]["passed"] and ref_row["full"]["p50_ms"] > 0


def test_nsight_commands_always_leave_clocks_alone_and_stay_small():
    from mini_train_sys_b200.bench import nsight

    for name in nsight.registered():
        line = nsight.command_for(name, "scripts/bench_ops.py", mode="full", output="x")
        assert "--clock-control none" in line and " && ncu " in line and "-c 3" in line
    with pytest.raises(ValueError):
        nsight.build_command(["x.py"], mode="full", kernel_regex="k", count=50)
    with pytest.raises(ValueError):
        nsight.build_command(["x.py"], mode="full")
    cmd = nsight.build_command(["x.py"], mode="launches", output="l.csv")
    assert cmd[:3] == ["ncu", "--clock-control", "none"] and "gpu__time_duration.sum" in cmd


def test_nsight_parsers():
    from mini_train_sys_b200.bench import nsight

    raw = '"ID","Kernel Name","gpu__time_duration.sum","dram__bytes_read.sum"\n"","","us","Mbyte"\n"0","k(int)","12.5","100"\n'
    rows = nsight.parse_raw_csv(raw)
    assert rows[0]["Kernel Name"] == "k(int)" and rows[0]["gpu__time_duration.sum [us]"] == "12.5"
    assert "duration" in nsight.roofline_summary(rows)
    listing = ('==PROF== x\n"ID","Process ID","Kernel Name","Metric Name","Metric Unit","Metric Value"\n'
               '"0","1","a(int)","gpu__time_duration.sum","ns","3000"\n"1","1","b()","gpu__time_duration.sum","ns","1000"\n'
               '"2","1","a(int)","gpu__time_duration.sum","ns","1000"\n')
    shares = nsight.launch_shares(nsight.parse_launch_list(listing))
    assert shares[0][0] == "a" and shares[0][1] == 2 and shares[0][3] == pytest.approx(0.8)


def _rows(world, tps, batch=8, status="ok", ops="torch", dispatch=None):
    return {"status": status, "strategy": "fsdp", "engine": "nccl", "ops": ops, "batch_size": batch, "world_size": world,
            "tokens_per_sec": tps, "step_ms_mean": 1.0, "data_stall_fraction": 0.01, "peak_reserved_mb_max": 10.0,
            "peak_allocated_mb_max": 5.0 + batch, "device_memory_mb": 100.0, "dispatch": dispatch}


def test_weak_table_capacity_choice_and_gates():
    from mini_train_sys_b200.bench import distributed as db

    rows = [_rows(1, 100.0), _rows(1, 100.0), _rows(2, 190.0), _rows(2, 186.0)]
    weak = db.weak_scaling_table(rows)
    two = next(w for w in weak if w["world_size"] == 2)
    assert two["efficiency_pct"] == pytest.approx(94.0)
    gates = db.quality_gates({"rows": rows, "weak": weak}, repeats=2)
    assert gates["passed"] and gates["min_efficiency_pct"] == pytest.approx(94.0)
    assert not db.quality_gates({"rows": rows + [_rows(2, 0, status="failed")], "weak": weak}, repeats=2)["passed"]

    cap_rows = [_rows(1, 100.0, batch=8), _rows(1, 101.0, batch=8), _rows(1, 150.0, batch=16), _rows(1, 151.0, batch=16),
                _rows(1, 140.0, batch=32), _rows(1, 139.0, batch=32), _rows(1, 500.0, batch=64)]
    cap = db.present_capacity(cap_rows)
    assert cap["selected"][0]["batch_size"] == 16 and not cap["selected"][0]["selected_is_largest_tested"]
    assert cap["selected"][0]["activation_mb_per_sample"] == pytest.approx(1.0)
    assert any(r["batch_size"] == 64 and r["reason"] == "repeats" for r in cap["rejected"])

    back = db.present_backend([_rows(1, 100.0), _rows(1, 100.0),
                               _rows(1, 300.0, ops="native", dispatch={"attention:native": 4}),
                               _rows(1, 300.0, ops="native", dispatch={"attention:native": 4, "attention:fallback": 1})])
    native = next(b for b in back if b["ops"] == "native")
    assert native["speedup_vs_torch"] == pytest.approx(3.0) and not native["valid"]


def test_weak_suite_end_to_end_on_gloo(tmp_path):
    cmd = [sys.executable, str(ROOT / "scripts" / "run_dist_bench.py"), "run", "--suite", "weak", "--config",
           str(ROOT / "configs" / "bench" / "debug_moe.yaml"), "--output-dir", str(tmp_path), "--strategies", "ddp",
           "--world-sizes", "1,2", "--ops-backends", "torch", "--engines", "nccl", "--batch-sizes", "4", "--repeats", "1",
           "--warmup-steps", "1", "--measure-steps", "3", "--master-port", "29643", "--timeout", "600"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    summary = json.loads((tmp_path / "weak" / "summary.json").read_text())
    assert all(r["status"] == "ok" for r in summary["rows"]), summary["rows"]
    assert {w["world_size"] for w in summary["weak"]} == {1, 2}
    assert (tmp_path / "weak" / "inventory.json").exists()
    # a second invocation reuses both results (identical identity hash)
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900)
    again = json.loads((tmp_path / "weak" / "summary.json").read_text())
    assert all(r.get("reused") for r in again["rows"])


def test_evidence_tooling_roundtrip(tmp_path):
    """Catalogue, audit and manifest of a small results tree; the manifest check notices a changed file."""

    tree = tmp_path / "results"
    raw = tree / "distributed" / "weak" / "raw"
    raw.mkdir(parents=True)
    rows = []
    for world, tps in ((1, 100.0), (2, 190.0)):
        row = {**_rows(world, tps), "name": f"r{world}", "identity": f"id{world}", "timing": "cuda events per step, max over ranks",
               "warmup_steps": 3}
        (raw / f"r{world}.json").write_text(json.dumps(row))
        rows.append(row)
    from mini_train_sys_b200.bench.distributed import weak_scaling_table

    (tree / "distributed" / "weak" / "summary.json").write_text(json.dumps({"suite": "weak", "rows": rows, "weak": weak_scaling_table(rows),
                                                                           "quality_gates": {"passed": True}}))
    (tree / "bench.json").write_text(json.dumps({"metric": "tokens/sec", "value": 1.0, "n_gpus": 1}))
    run = lambda *a: subprocess.run([sys.executable, *a], capture_output=True, text=True, timeout=300)   # noqa: E731
    out = run(str(ROOT / "scripts" / "build_results_catalog.py"), str(tree))
    assert out.returncode == 0 and json.loads(out.stdout)["kinds"] == {"distributed/weak": 1, "bench": 1, "json": 2}, out.stdout + out.stderr
    assert run(str(ROOT / "scripts" / "audit_results_export.py"), str(tree)).returncode == 0
    # a path of the machine inside an exported file: a warning, a failure only when asked for; URLs and relative paths are fine
    (tree / "note.md").write_text("config /home/someone/run.yaml, see https://example.org/home/page and results/operators/a.json\n")
    lenient = run(str(ROOT / "scripts" / "audit_results_export.py"), str(tree))
    assert lenient.returncode == 0 and json.loads(lenient.stdout)["non_portable"] == ["note.md: /home/someone"]
    assert run(str(ROOT / "scripts" / "audit_results_export.py"), str(tree), "--strict-paths").returncode == 1
    (tree / "note.md").unlink()
    assert run(str(ROOT / "scripts" / "build_results_manifest.py"), str(tree)).returncode == 0
    assert run(str(ROOT / "scripts" / "build_results_manifest.py"), str(tree), "--check").returncode == 0
    (tree / "bench.json").write_text("{}")
    bad = run(str(ROOT / "scripts" / "build_results_manifest.py"), str(tree), "--check")
    assert bad.returncode == 1 and "bench.json" in bad.stdout
    rows[1]["identity"] = "tampered"
    (tree / "distributed" / "weak" / "summary.json").write_text(json.dumps({"suite": "weak", "rows": rows, "weak": weak_scaling_table(rows)}))
    assert run(str(ROOT / "scripts" / "audit_results_export.py"), str(tree)).returncode == 1


def test_operator_plots_are_well_formed_and_complete(tmp_path):
    import xml.etree.ElementTree as ET

    from mini_train_sys_b200.bench.plots import kernel_grid_svg, write_kernel_plots

    table = []
    for tokens in (512, 2048, 8192):
        table.append({"kernel": "rmsnorm", "profile": "p", "tokens": tokens, "provider": "torch", "fwd_ms": tokens / 1000, "full_ms": tokens / 400,
                      "bwd_ms": tokens / 700, "speedup_full": 1.0})
        table.append({"kernel": "rmsnorm", "profile": "p", "tokens": tokens, "provider": "native", "fwd_ms": tokens / 9000, "full_ms": tokens / 4000,
                      "bwd_ms": None, "speedup_full": 10.0})
    table.append({"kernel": "rope", "profile": "p", "tokens": 512, "provider": "native", "fwd_ms": 0.1, "full_ms": 0.2, "bwd_ms": 0.1, "speedup_full": None})
    svg = kernel_grid_svg(table, "rmsnorm")
    root = ET.fromstring(svg)
    ns = "{http://www.w3.org/2000/svg}"
    assert len(root.findall(f"{ns}polyline")) == 2 + 2 + 1 + 2          # backward of `native` has no data
    assert svg.count("<circle") == 3 * (2 + 2 + 1 + 2) and "stroke-dasharray" in svg and ">8192<" in svg
    written = write_kernel_plots(table, tmp_path / "plots")
    assert written == ["rmsnorm.svg", "rope.svg"] and "no data" in (tmp_path / "plots" / "rope.svg").read_text()
    # the summarize command writes them from cached scans
    cache = tmp_path / "scan"
    cache.mkdir()
    rows = [{"kernel": "swiglu", "tokens": t, "provider": pr, "fwd": {"p50_ms": 0.1 * t / 512}, "full": {"p50_ms": 0.3 * t / 512},
             "bwd": {"p50_ms": 0.2 * t / 512}} for t in (512, 1024) for pr in ("torch", "native")]
    (cache / "x.json").write_text(json.dumps({"k": {"status": "ok", "profile": "p", "rows": rows}}))
    out = subprocess.run([sys.executable, str(ROOT / "scripts" / "bench_ops.py"), "summarize", str(cache), "--plots", str(tmp_path / "p2")],
                         capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    assert (tmp_path / "p2" / "swiglu.svg").is_file() and '"plots": ["swiglu.svg"]' in out.stdout


def test_capacity_ladder_comes_from_the_memory_plan():
    from mini_train_sys_b200.bench.distributed import planned_batch_ladder

    config = str(ROOT / "configs" / "bench" / "synbios_moe_fsdp.yaml")
    ladder = planned_batch_ladder(config, None, strategies=("fsdp",), world_sizes=(1, 8))
    assert ladder == tuple(sorted(set(ladder))) and len(ladder) >= 5 and all(b % 8 == 0 for b in ladder)
    assert 500 < ladder[-1] < 800 and ladder[0] <= ladder[-1] // 8 + 8           # brackets the planned limit of a 180 GiB device from below
    small = planned_batch_ladder(config, None, strategies=("fsdp",), world_sizes=(1, 8), device_gib=40.0)
    assert small[-1] < ladder[-1] / 4
    with pytest.raises(ValueError):
        planned_batch_ladder(config, None, strategies=("fsdp",), world_sizes=(1,), device_gib=2.0)     # not even the resident part fits
    import importlib.util

    spec = importlib.util.spec_from_file_location("run_dist_bench", ROOT / "scripts" / "run_dist_bench.py")
    cli = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cli)
    args = cli._parser().parse_args(["run", "--suite", "capacity", "--batch-sizes", "auto"])
    assert args.batch_sizes == "auto" and cli._parser().parse_args(["run", "--suite", "weak", "--batch-sizes", "8,16"]).batch_sizes == (8, 16)


def test_distributed_benchmark_cli_takes_the_reference_spellings(tmp_path, capsys):
    """Space-separated lists, ``--output`` / ``--case-config`` / ``--local-batch`` on ``run``; ``--input`` / ``--output`` and the
    capacity limits on the presenters; a failed validation verdict blocks ``present-backend``."""

    import importlib.util

    spec = importlib.util.spec_from_file_location("run_dist_bench", ROOT / "scripts" / "run_dist_bench.py")
    cli = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(cli)
    args = cli._parser().parse_args(["run", "--suite", "weak", "--world-sizes", "1", "2", "4", "--strategies", "ddp", "fsdp", "--ops-backends",
                                     "torch,native", "--batch-sizes", "8", "16", "--output", "out", "--case-config", "c.yaml", "--local-batch", "4",
                                     "--case-timeout-seconds", "60"])
    assert (args.world_sizes, args.strategies, args.ops_backends, args.batch_sizes) == ((1, 2, 4), ("ddp", "fsdp"), ("torch", "native"), (8, 16))
    assert (args.output_dir, args.config, args.local_batch, args.timeout) == ("out", "c.yaml", 4, 60.0)

    from mini_train_sys_b200.bench import distributed as db

    rows = [_rows(1, 100.0, batch=1), _rows(1, 101.0, batch=1), _rows(1, 150.0, batch=16), _rows(1, 151.0, batch=16), _rows(1, 500.0, batch=64)]
    suite_dir = tmp_path / "capacity"
    suite_dir.mkdir()
    (suite_dir / "summary.json").write_text(json.dumps({"suite": "capacity", "rows": rows, "capacity": db.present_capacity(rows),
                                                       "quality_gates": {"passed": True}}))
    table = tmp_path / "tables" / "capacity.md"
    assert cli.main(["present-capacity", "--input", str(suite_dir / "summary.json"), "--output", str(table), "--require-batch-one"]) == 0
    assert "common fixed batch: 16" in table.read_text() and "| 16 |" in table.read_text()
    # one repeat is enough under --min-repeats 1, so the single row at 64 now wins; the directory form of --input works too
    assert cli.main(["present-capacity", "--input", str(suite_dir), "--min-repeats", "1", "--output", str(table)]) == 0
    assert "common fixed batch: 64" in table.read_text()
    no_one = [r for r in rows if r["batch_size"] != 1]
    (suite_dir / "summary.json").write_text(json.dumps({"suite": "capacity", "rows": no_one, "capacity": db.present_capacity(no_one),
                                                       "quality_gates": {"passed": True}}))
    assert cli.main(["present-capacity", str(tmp_path), "--require-batch-one"]) == 1

    back_rows = [_rows(1, 100.0), _rows(1, 100.0), _rows(1, 300.0, ops="native", dispatch={"attention:native": 4}),
                 _rows(1, 300.0, ops="native", dispatch={"attention:native": 4})]
    (tmp_path / "backend").mkdir()
    (tmp_path / "backend" / "summary.json").write_text(json.dumps({"suite": "backend", "rows": back_rows, "backend": db.present_backend(back_rows),
                                                                  "quality_gates": {"passed": True}}))
    verdict = tmp_path / "validation.json"
    verdict.write_text(json.dumps({"passed": False}))
    assert cli.main(["present-backend", "--input", str(tmp_path / "backend"), "--validation", str(verdict)]) == 1
    verdict.write_text(json.dumps({"passed": True}))
    assert cli.main(["present-backend", "--input", str(tmp_path / "backend"), "--validation", str(verdict), "--output", str(tmp_path / "b.md")]) == 0
    assert "speedup_vs_torch" in (tmp_path / "b.md").read_text()

    assert cli.main(["inventory", "--output", str(tmp_path / "inv")]) == 0
    assert "source_fingerprint" in json.loads((tmp_path / "inv" / "inventory.json").read_text())
    capsys.readouterr()
