"""SynBioS interventions and reports on CPU: byte codec, tiny MoE model, a handful of probe steps."""

import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
CLI = [sys.executable, str(ROOT / "scripts" / "synbios_moe.py")]
MODEL = {"vocab_size": 257, "seq_len": 512, "n_layers": 2, "n_heads": 2, "hidden_size": 32, "intermediate_size": 32,
         "ffn_type": "moe", "num_experts": 4, "experts_per_token": 2, "dropout": 0.0}


def run(*args, timeout=900):
    done = subprocess.run([*CLI, *args], capture_output=True, text=True, timeout=timeout)
    assert done.returncode == 0, done.stdout[-1500:] + done.stderr[-2500:]
    return done.stdout


@pytest.fixture(scope="module")
def studies(tmp_path_factory):
    """Two matched studies (single, multi5+permute) of the same 20 people, each with the probe heads the mechanisms need."""

    root = tmp_path_factory.mktemp("mechanisms")
    (root / "model.yaml").write_text(json.dumps({"model": MODEL}))
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend

    torch.manual_seed(0)
    model = MiniTransformer(ModelConfig(**MODEL), get_ops_backend("torch"), activation_dtype=torch.float32)
    torch.save(model.state_dict(), root / "model.pt")
    out = {"root": root, "model_config": str(root / "model.yaml"), "checkpoint": str(root / "model.pt")}
    base = ["--model-config", out["model_config"], "--checkpoint", out["checkpoint"], "--codec", "bytes", "--device", "cpu", "--quiet"]
    for condition, variant in (("single", "single"), ("multi5_permute", "multi5+permute")):
        data, cache, probes = root / condition / "data", root / condition / "cache", root / condition / "probes"
        run("prepare", "--output", str(data), "--variant", variant, "--num-people", "20", "--codec", "bytes", "--quiet")
        run("cache-probes", "--data", str(data), "--output", str(cache), "--codec", "bytes")
        for kind, attribute, target in (("q", "university", "first"), ("q", "university", "whole"), ("p", "university", "first"),
                                        ("p", "university", "whole")):
            run("probe", *base, "--data", str(data), "--probe-cache", str(cache), "--kind", kind, "--attribute", attribute,
                "--target", target, "--steps", "3", "--batch-size", "4", "--evaluate-train",
                "--output", str(probes / "training" / f"{kind}-{attribute}-{target}.json"))
        out[condition] = {"data": data, "cache": cache, "probes": probes}
    out["base"] = base
    return out


def test_insertion_and_summary_arithmetic():
    from experiments.synbios_moe.mechanisms.oracle_first_token import insert_oracle_first_token, summarize_oracle_rows

    assert insert_oracle_first_token([256, 10, 11, 256], 32, 256) == [256, 10, 11, 32, 256]
    with pytest.raises(ValueError):
        insert_oracle_first_token([256, 10, 11], 32, 256)
    rows = [{"whole_before_correct": b, "whole_after_correct": a} for b, a in ((0, 1), (0, 0), (0, 1), (1, 1), (1, 0))]
    s = summarize_oracle_rows(rows)
    assert s["examples"] == 5 and s["baseline_errors"] == 3 and s["recovered_errors"] == 2 and s["harmed_correct"] == 1
    assert s["recovery_rate"] == pytest.approx(2 / 3) and s["harm_rate"] == 0.5 and s["accuracy_delta"] == pytest.approx(0.2)
    assert summarize_oracle_rows([])["accuracy_before"] == 0.0


def test_oracle_first_token_runs_on_unchanged_heads(studies):
    s = studies["multi5_permute"]
    out = studies["root"] / "oracle"
    run("oracle-first-token", *studies["base"], "--data", str(s["data"]), "--probe-cache", str(s["cache"]), "--probe-dir", str(s["probes"]),
        "--output", str(out), "--attributes", "university", "--batch-size", "7")
    summary = json.loads((out / "summary.json").read_text())
    assert summary["protocol"] == "q_whole_oracle_first_token_v1" and summary["parameters_updated"] is False
    held_out = int((np.load(s["cache"] / "profile_splits.npy") == 1).sum())
    assert summary["overall"]["examples"] == held_out == summary["attributes"][0]["examples"]
    records = (out / "records.csv").read_text().splitlines()
    assert len(records) == held_out + 1 and "whole_after_correct" in records[0]


def test_ground_truth_first_inputs_and_training(studies, tmp_path):
    from experiments.synbios_moe.codec import get_codec
    from experiments.synbios_moe.mechanisms.first_token_intervention import (GroundTruthFirstWholeDataset, build_ground_truth_first_input,
                                                                             first_token_text, prepare_ground_truth_first_whole_data)
    from experiments.synbios_moe.probes.dataset import CachedProbeDataset, ProbeItem

    codec = get_codec("bytes")
    assert first_token_text("32", codec) == (32, " ")
    for bad in ("x", "256", "65"):          # not an id, the EOS, no leading space
        with pytest.raises(ValueError):
            first_token_text(bad, codec)
    item = ProbeItem(np.arange(20), np.asarray([2, 5, 8, 11, 14, 17]), 3)
    rebuilt = build_ground_truth_first_input(item, 1, 99)
    assert rebuilt.input_ids.tolist() == [0, 1, 2, 3, 4, 5, 99] and rebuilt.positions.tolist() == [6] and rebuilt.label == 3
    s = studies["multi5_permute"]
    prepared = prepare_ground_truth_first_whole_data(cache_root=s["cache"], probe_dir=s["probes"], attribute="university", codec=codec)
    whole = CachedProbeDataset(s["cache"], kind="p", attribute="university", target="whole", split="train")
    data = prepared.train_data
    assert isinstance(data, GroundTruthFirstWholeDataset) and len(data) == 6 * len(whole) and prepared.rank == 2
    sample = data[7]                                         # source 1, position 1
    src = whole[1]
    assert sample.label == src.label and sample.input_ids[-1] == 32
    assert sample.input_ids[:-1].tolist() == src.input_ids[: src.positions[1] + 1].tolist()
    assert max(len(i.input_ids) for i in data.longest(3)) == max(len(data[i].input_ids) for i in range(len(data)))
    with pytest.raises(ValueError):
        prepare_ground_truth_first_whole_data(cache_root=s["cache"], probe_dir=s["probes"], attribute="birth_date", codec=codec)
    # the CLI trains it (resumable) and the report joins it with the original P probes
    out = tmp_path / "gtf"
    run("ground-truth-first-whole", *studies["base"], "--probe-cache", str(s["cache"]), "--probe-dir", str(s["probes"]),
        "--attribute", "university", "--steps", "3", "--batch-size", "4", "--output", str(out / "university.json"))
    rec = json.loads((out / "university.json").read_text())
    assert rec["protocol"] == "ground_truth_first_whole_rank_matched_v1" and len(rec["whole_accuracy_validation_by_source_position"]) == 6
    assert sum(rec["whole_total_validation_by_source_position"]) == 6 * len(prepared.validation_data.whole_data)
    assert (out / "university.pt").is_file()
    run("ground-truth-first-report", "--run-dir", str(out), "--probe-dir", str(s["probes"]), "--output", str(out / "report"))
    summary = json.loads((out / "report" / "summary.json").read_text())
    assert summary["attributes_reported"] == ["university"] and "major" in summary["attributes_missing"]
    assert "| university |" in (out / "report" / "report.md").read_text()


def test_exposure_curve_fit_recovers_known_parameters(tmp_path):
    from experiments.synbios_moe.mechanisms.company_relation import fit_company_pair, fit_exposure_curve, load_position_curves, paired_exposure
    from experiments.synbios_moe.pretraining.dataset import WHOLE_ATTRIBUTES

    x = paired_exposure()
    assert x.tolist() == pytest.approx([0.0, 1 / 3, 0.6, 0.8, 14 / 15, 1.0])
    fit = fit_exposure_curve(0.2 + 0.7 * x, x)
    assert fit["baseline"] == pytest.approx(0.2) and fit["gain"] == pytest.approx(0.7) and fit["rmse"] < 1e-12
    assert fit["saturation"] == pytest.approx(0.9) and fit["leave_one_out_rmse"] < 1e-10
    rows = ["condition,split,kind,target,attribute,position,accuracy"]
    for attribute in WHOLE_ATTRIBUTES:
        gain = 0.6 if attribute in ("company", "company_city") else 0.05
        rows += [f"multi5_permute,person_held_out_validation,p,whole,{attribute},{k},{0.1 + gain * x[k]}" for k in range(6)]
        rows += [f"single,person_held_out_validation,p,whole,{attribute},{k},0.0" for k in range(6)]
    (tmp_path / "tidy.csv").write_text("\n".join(rows) + "\n")
    summary = fit_company_pair(load_position_curves(tmp_path / "tidy.csv", condition="multi5_permute"), tmp_path / "out")
    assert summary["pair_mean_gain"] == pytest.approx(0.6) and summary["unpaired_max_gain"] == pytest.approx(0.05)
    assert (tmp_path / "out" / "company_relation_metrics.csv").read_text().count("\n") == 6
    with pytest.raises(ValueError):
        load_position_curves(tmp_path / "tidy.csv", condition="nothing")


def test_probe_batch_benchmark_and_merge(studies, tmp_path):
    s = studies["multi5_permute"]
    a, b = tmp_path / "gpu0.json", tmp_path / "gpu1.json"
    for out in (a, b):
        run("probe-batch-benchmark", *studies["base"], "--probe-cache", str(s["cache"]), "--attribute", "university", "--target", "whole",
            "--p-batch-sizes", "2,4", "--q-batch-sizes", "2,4", "--warmup-steps", "1", "--measure-steps", "2", "--output", str(out))
    rec = json.loads(a.read_text())
    assert [r["kind"] for r in rec["benchmarks"]] == ["p", "q"]
    for bench in rec["benchmarks"]:
        assert [r["batch_size"] for r in bench["results"]] == [2, 4] and all(r["status"] == "completed" for r in bench["results"])
        assert bench["recommended_capacity_batch_size"] in (2, 4)
    run("summarize-probe-batch-benchmarks", str(a), str(b), "--output", str(tmp_path / "merged.json"))
    merged = json.loads((tmp_path / "merged.json").read_text())
    assert merged["recommendations"]["p_training"]["replicas"] == 2 and merged["recommendations"]["q_training"]["recommended_batch_size"] in (2, 4)
    # validation cells were not measured, so the merge is not ready for a formal run and no environment file is written
    assert merged["completeness"]["missing"] == ["p_validation", "q_validation"] and not merged["completeness"]["ready_for_formal"]
    from experiments.synbios_moe.probes.batch_benchmark import parse_batch_sizes, probe_batch_environment, summarize_probe_benchmarks

    with pytest.raises(ValueError, match="not complete"):
        probe_batch_environment(merged)

    def result(kind, mode, speeds, limit=92.0, **identity):
        return {"kind": kind, "mode": mode, "memory_limit_percent": limit, **identity,
                "results": [{"batch_size": b, "status": "completed", "examples_per_second": v, "peak_memory_percent": 10.0 * n}
                            for n, (b, v) in enumerate(speeds.items(), start=1)]}

    paths = []
    for replica in range(2):
        for kind in ("p", "q"):
            for mode in ("training", "validation"):
                path = tmp_path / f"{kind}-{mode}-{replica}.json"
                path.write_text(json.dumps(result(kind, mode, {8: 100.0, 16: 180.0 + replica, 32: 150.0}, attribute="university")))
                paths.append(path)
    full = summarize_probe_benchmarks(paths)
    assert full["completeness"]["ready_for_formal"] and full["recommendations"]["q_validation"]["recommended_batch_size"] == 16
    assert probe_batch_environment(full) == ("export P_BATCH_SIZE=16\nexport Q_BATCH_SIZE=16\nexport P_VALIDATION_BATCH_SIZE=16\n"
                                             "export Q_VALIDATION_BATCH_SIZE=16\n")
    # the best candidate at the edge of the search, replicas that tried different candidates, limits or tasks: all flagged or refused
    edge = tmp_path / "edge.json"
    edge.write_text(json.dumps(result("p", "training", {8: 100.0, 16: 180.0, 32: 250.0}, attribute="university")))
    assert summarize_probe_benchmarks([edge])["completeness"]["at_search_boundary"] == ["p_training"]
    other = tmp_path / "other.json"
    other.write_text(json.dumps(result("p", "training", {8: 100.0, 16: 180.0}, attribute="university")))
    with pytest.raises(ValueError, match="different batch-size candidates"):
        summarize_probe_benchmarks([paths[0], other])
    other.write_text(json.dumps(result("p", "training", {8: 100.0, 16: 180.0, 32: 150.0}, limit=80.0, attribute="university")))
    with pytest.raises(ValueError, match="memory limits"):
        summarize_probe_benchmarks([paths[0], other])
    other.write_text(json.dumps(result("p", "training", {8: 100.0, 16: 180.0, 32: 150.0}, attribute="major")))
    with pytest.raises(ValueError, match="disagree on attribute"):
        summarize_probe_benchmarks([paths[0], other])
    env = tmp_path / "batch.env"
    run("summarize-probe-benchmarks", *[a for p_ in paths for a in ("--run", str(p_))], "--output", str(tmp_path / "m2.json"),
        "--env-output", str(env), "--require-complete-search")
    assert env.read_text().startswith("export P_BATCH_SIZE=16")
    done = subprocess.run([*CLI, "summarize-probe-benchmarks", str(a), str(b), "--output", str(tmp_path / "m3.json"), "--require-complete-search"],
                          capture_output=True, text=True)
    assert done.returncode == 2 and "benchmark incomplete" in done.stderr

    assert parse_batch_sizes("8, 2,8,4") == (2, 4, 8)
    with pytest.raises(ValueError):
        parse_batch_sizes("4,0")


def test_formal_comparison_requires_matched_complete_studies(studies, tmp_path):
    from experiments.synbios_moe.probes import comparison_report as cr

    # a complete study: every one of the 22 heads present (copies of the trained ones with the identity rewritten)
    def complete(condition):
        src = studies[condition]["probes"]
        dst = tmp_path / condition
        (dst / "training").mkdir(parents=True)
        from experiments.synbios_moe.probes.dataset import probe_tasks

        jobs = {}
        for kind in ("p", "q"):
            template = json.loads((src / "training" / f"{kind}-university-whole.json").read_text())
            for t in probe_tasks():
                rec = json.loads(json.dumps(template))
                rec["identity"].update({"kind": kind, "attribute": t.attribute, "target": t.target})
                name = f"{kind}-{t.attribute}-{t.target}"
                (dst / "training" / f"{name}.json").write_text(json.dumps(rec))
                jobs[name] = {"status": "done", "phase": "training"}
        (dst / "pipeline.json").write_text(json.dumps({"identity": "x", "jobs": jobs}))
        return dst

    single, multi = complete("single"), complete("multi5_permute")
    out = tmp_path / "report"
    run("compare-formal-studies", "--single", str(single), "--multi", str(multi), "--single-cache", str(studies["single"]["cache"]),
        "--multi-cache", str(studies["multi5_permute"]["cache"]), "--output", str(out))
    head = json.loads((out / "headline_metrics.json").read_text())
    assert set(head) == {"single", "multi5_permute", "delta_multi_minus_single", "published_q_reference_macro_means"}
    assert len(head["single"]) == 6
    tidy = (out / "probe_metrics_tidy.csv").read_text().splitlines()
    # 2 conditions x (11 P heads x 6 + 11 Q heads x 1) positions x 2 splits (validation and train recall)
    assert len(tidy) - 1 == 2 * (11 * 6 + 11) * 2
    # figures: labelled SVG grids (one value per attribute and position) with PNG twins, and the overview bars
    figures = sorted(f.name for f in (out / "figures").iterdir())
    assert figures == sorted(["overview.svg", "p_first_heatmaps.svg", "p_whole_heatmaps.svg", "q_first_table.svg", "q_whole_table.svg",
                              "p_first_single.png", "p_first_multi5_permute.png", "p_whole_single.png", "p_whole_multi5_permute.png"])
    svg = (out / "figures" / "p_first_heatmaps.svg").read_text()
    assert svg.startswith("<svg") and svg.count("<rect") >= 2 * 36 and "birth date" in svg and ">P5<" in svg
    assert (out / "figures" / "p_whole_single.png").read_bytes()[:8] == b"\x89PNG\r\n\x1a\n"
    assert "figures/overview.svg" in (out / "report.md").read_text()
    # swapped conditions, different people and different hyper-parameters are all refused
    a = cr.load_formal_run("single", single, studies["single"]["cache"])
    b = cr.load_formal_run("multi5_permute", multi, studies["multi5_permute"]["cache"])
    cr.validate_matched_runs(a, b)
    with pytest.raises(ValueError, match="variant"):
        cr.validate_matched_runs(cr.load_formal_run("single", multi, studies["multi5_permute"]["cache"]), b)
    rec = json.loads((multi / "training" / "q-major-whole.json").read_text())
    rec["identity"]["steps"] = 99
    (multi / "training" / "q-major-whole.json").write_text(json.dumps(rec))
    with pytest.raises(ValueError, match="steps differs"):
        cr.validate_matched_runs(a, cr.load_formal_run("multi5_permute", multi, studies["multi5_permute"]["cache"]))
    (multi / "training" / "q-major-whole.json").unlink()
    with pytest.raises(ValueError, match="no training result"):
        cr.load_formal_run("multi5_permute", multi, studies["multi5_permute"]["cache"])


def test_diagnostic_report_checks_its_inputs(studies, tmp_path):
    roots = {}
    for condition in ("single", "multi5_permute"):
        s = studies[condition]
        out = tmp_path / condition
        run("oracle-first-token", *studies["base"], "--data", str(s["data"]), "--probe-cache", str(s["cache"]), "--probe-dir", str(s["probes"]),
            "--output", str(out / "oracle"), "--attributes", "university")
        run("analyze", *studies["base"], "--data", str(s["data"]), "--output", str(out / "routes.json"), "--max-items", "8")
        roots[condition] = out
    summary = json.loads(run("diagnostic-report", "--single", str(roots["single"]), "--multi", str(roots["multi5_permute"]),
                             "--output", str(tmp_path / "diag")))
    assert summary["route_layers"] == 2 and set(summary["oracle_overall"]) == {"single", "multi5_permute"}
    assert "nmi_attribute_expert_delta" in (tmp_path / "diag" / "routes_by_layer.csv").read_text().splitlines()[0]
    # an edited summary (overall row no longer the mean of its attribute rows) is refused
    path = roots["single"] / "oracle" / "summary.json"
    rec = json.loads(path.read_text())
    rec["overall"]["examples"] += 1
    path.write_text(json.dumps(rec))
    from experiments.synbios_moe.mechanisms.comparison_report import load_diagnostic_evidence

    with pytest.raises(ValueError, match="cover"):
        load_diagnostic_evidence(roots)


def test_two_condition_audit_writes_lineage_and_notices_tampering(studies, tmp_path):
    args = []
    for side, condition in (("single", "single"), ("multi", "multi5_permute")):
        s = studies[condition]
        args += [f"--{side}-data", str(s["data"]), f"--{side}-cache", str(s["cache"]), f"--{side}-model", studies["checkpoint"]]
    out = json.loads(run("audit-synbios-repository", *args, "--output", str(tmp_path / "audit")))
    assert out["status"] == "passed" and out["checks"] >= 6
    lineage = json.loads((tmp_path / "audit" / "dataset_lineage.json").read_text())
    for condition in ("single", "multi5_permute"):
        rec = lineage[condition]
        assert rec["token_shards"]["documents"] == rec["source_dataset"]["biographies"]          # one document per biography
        assert rec["probe_cache"]["parent_manifest_sha256"] == rec["source_dataset"]["manifest_sha256"]
        assert (studies[condition]["data"] / "lineage.json").is_file() and (studies[condition]["cache"] / "lineage.json").is_file()
    assert lineage["single"]["source_dataset"]["profiles_sha256"] == lineage["multi5_permute"]["source_dataset"]["profiles_sha256"]
    # a shard that changed after the manifest was written is found
    shard = studies["single"]["data"] / "token_shards" / "train" / "shard_00000.bin"
    original = shard.read_bytes()
    try:
        shard.write_bytes(original[:-2] + b"\x01\x00")
        done = subprocess.run([*CLI, "audit-synbios-repository", *args, "--output", str(tmp_path / "audit2")], capture_output=True, text=True)
        assert done.returncode == 1 and "shard_00000.bin differs" in done.stdout
    finally:
        shard.write_bytes(original)


def test_pairwise_branching_separates_token_driven_routes():
    """Synthetic cases: the route at t1 depends on t1 only, the route at t2 on t2 only.  Same-t2 pairs then overlap fully at both
    positions, different-t2 pairs fully at t1 and not at all at t2: branching scores 0 and 1."""

    from experiments.synbios_moe.mechanisms.token_routes import pairwise_branching

    route_of = {7: [0, 1], 8: [2, 3], 9: [4, 5]}
    cases = []
    for n in range(12):
        t2 = (7, 8, 9)[n % 3]
        cases.append({"attribute": "university", "t1_id": 40, "t2_id": t2, "routes": [[[6, 7], [6, 7]], [route_of[t2], route_of[t2]]]})
    rows = pairwise_branching(cases, layers=2, pair_limit=50, seed=3)
    by = {(r["layer"], r["pair_group"]): r for r in rows}
    assert set(by) == {(0, "same_t2"), (0, "different_t2"), (1, "same_t2"), (1, "different_t2")}
    for layer in (0, 1):
        assert by[(layer, "same_t2")]["branching_score"] == 0.0 and by[(layer, "same_t2")]["t2_route_overlap"] == 1.0
        assert by[(layer, "different_t2")]["t1_route_overlap"] == 1.0 and by[(layer, "different_t2")]["branching_score"] == 1.0
        assert by[(layer, "different_t2")]["pair_count"] == 50
    # one t2 group only: nothing to contrast, and a single member gives no same-t2 pair either
    assert pairwise_branching(cases[:1], layers=2) == []


def test_routes_at_positions_match_a_full_capture():
    from experiments.synbios_moe.mechanisms.routing import routes_for_batch
    from experiments.synbios_moe.mechanisms.token_routes import routes_at_positions
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend

    torch.manual_seed(1)
    model = MiniTransformer(ModelConfig(**MODEL), get_ops_backend("torch"), activation_dtype=torch.float32).eval()
    ids = torch.randint(0, 256, (3, 11))
    pos = torch.tensor([[2, 3], [5, 6], [9, 10]])
    got = routes_at_positions(model, ids, pos)
    full = routes_for_batch(model, ids)
    assert got.shape == (3, 2, MODEL["n_layers"], MODEL["experts_per_token"])
    for b in range(3):
        for j in range(2):
            for layer in range(MODEL["n_layers"]):
                assert got[b, j, layer].tolist() == full[layer][b, int(pos[b, j])].tolist()
    dense = MiniTransformer(ModelConfig(**{**MODEL, "ffn_type": "dense"}), get_ops_backend("torch"), activation_dtype=torch.float32)
    with pytest.raises(ValueError, match="routed experts"):
        routes_at_positions(dense, ids, pos)


def test_bad_case_routes_command_writes_the_protocol_files(studies):
    s = studies["multi5_permute"]
    out = studies["root"] / "bad_case_routes"
    run("validate-probe-bad-case-routes", *studies["base"], "--data", str(s["data"]), "--probe-cache", str(s["cache"]),
        "--probe-dir", str(s["probes"]), "--output", str(out), "--attributes", "university", "--batch-size", "5", "--pair-limit", "20")
    summary = json.loads((out / "summary.json").read_text())
    assert summary["protocol"] == "q_bad_case_t1_t2_route_branching_v1" and summary["parameters_updated"] is False
    assert summary["experts"] == MODEL["num_experts"] and summary["top_k"] == 2
    cases = (out / "bad_cases.csv").read_text().splitlines()
    assert len(cases) == summary["examples"] + 1 == summary["attributes"]["university"] + 1
    records = (out / "route_records.csv").read_text().splitlines()
    assert len(records) - 1 == summary["examples"] * summary["layers"]
    for name in ("pairwise_branching.csv", "token_route_nmi.csv"):
        assert (out / name).is_file()


def test_bad_case_route_validation_on_forced_bad_cases(tmp_path, monkeypatch):
    """Predictions are injected (first token right, whole value wrong), so every record is a bad case: the routes recorded for it
    are those of the frozen backbone at the two value-token positions of ``[EOS] name t1 t2 [EOS]``."""

    from experiments.synbios_moe.codec import get_codec
    from experiments.synbios_moe.mechanisms import q_readout, token_routes
    from experiments.synbios_moe.mechanisms.routing import routes_for_batch
    from mini_train_sys_b200.models import MiniTransformer, ModelConfig, get_ops_backend

    codec = get_codec("bytes")
    torch.manual_seed(2)
    model = MiniTransformer(ModelConfig(**MODEL), get_ops_backend("torch"), activation_dtype=torch.float32).eval()
    values = ["MIT", "MIT", "Ohio", "Yale", "M"]          # byte codec: t1 is the space, t2 the first letter
    records = []
    for n, value in enumerate(values):
        name = codec.encode(f"Person {n}")
        records.append(q_readout.QPrediction(
            case_id=n, profile_index=n, person_id=f"p{n}", attribute="university", input_ids=(codec.eos, *name, codec.eos),
            true_first_id=0, pred_first_id=0, true_first_token=str(codec.encode(" " + value)[0]), pred_first_token="x",
            true_whole_id=1, pred_whole_id=2 if n != 3 else 1, true_whole_value=value, pred_whole_value="other",
            whole_true_probability=0.1))
    monkeypatch.setattr(q_readout, "collect_q_predictions", lambda *a, **k: (records, None))
    summary = token_routes.bad_case_route_validation(model, codec, data_root=tmp_path, cache_root=tmp_path, probe_dir=tmp_path,
                                                     output_dir=tmp_path / "out", attributes=("university",), batch_size=2, pair_limit=10)
    assert summary["examples"] == 4 and summary["layers"] == MODEL["n_layers"]          # the correctly read "Yale" is not a bad case
    import csv

    cases = list(csv.DictReader(open(tmp_path / "out" / "bad_cases.csv")))
    assert [c["true_whole_value"] for c in cases] == ["MIT", "MIT", "Ohio", "M"]
    first = records[0]
    t1, t2 = codec.encode(" MIT")[:2]
    ids = torch.tensor([[*first.input_ids[:-1], t1, t2, codec.eos]])
    full = routes_for_batch(model, ids)
    at = len(first.input_ids) - 1
    want_t1 = "|".join("+".join(str(e) for e in full[layer][0, at].tolist()) for layer in sorted(full))
    want_t2 = "|".join("+".join(str(e) for e in full[layer][0, at + 1].tolist()) for layer in sorted(full))
    assert cases[0]["t1_route_path"] == want_t1 and cases[0]["t2_route_path"] == want_t2
    assert cases[0]["t1_id"] == str(t1) and cases[0]["t2_text"] == codec.decode([t2])
    pairs = list(csv.DictReader(open(tmp_path / "out" / "pairwise_branching.csv")))
    assert {p["pair_group"] for p in pairs} == {"same_t2", "different_t2"}                  # MIT / MIT / M share t2, Ohio does not
    nmi = list(csv.DictReader(open(tmp_path / "out" / "token_route_nmi.csv")))
    assert len(nmi) == MODEL["n_layers"] and all(0.0 <= float(r["t1_top1_token_nmi"]) <= 1.0 + 1e-9 for r in nmi)


def test_figure_grids_carry_values_labels_and_outlines():
    from experiments.synbios_moe.probes import figures

    frag, w, h = figures.grid_svg([[0.0, 0.5], [1.0, 0.123]], row_labels=["a", "b & c"], col_labels=["P0", "P1"], title="t <1>",
                                  outlined=[(1, 0)])
    assert ">0.0<" in frag and ">50.0<" in frag and ">100.0<" in frag and ">12.3<" in frag
    assert "b &amp; c" in frag and "t &lt;1&gt;" in frag and frag.count("stroke-width='3'") == 1
    assert w == 130 + 2 * 64 and h == 34 + 2 * 64 + 28
    assert figures.accuracy_colour(-1.0) == figures.accuracy_colour(0.0) == (247, 251, 255)
    assert figures.accuracy_colour(2.0) == figures.accuracy_colour(1.0) == (8, 88, 110)
    with pytest.raises(ValueError):
        figures.grid_svg([[0.1]], row_labels=["a", "b"], col_labels=["x"], title="")
    png = figures.grid_png([[0.0, 1.0]], cell=4)
    assert png[:8] == b"\x89PNG\r\n\x1a\n" and int.from_bytes(png[16:20], "big") == 8 and int.from_bytes(png[20:24], "big") == 4
    head = {"single": {"a_b": 0.25, "c": 1.0}, "multi5_permute": {"a_b": 0.75, "c": 0.5}}
    bars = figures.overview_svg(head)
    assert bars.count("<rect") >= 1 + 4 + 2 and ">25.0<" in bars and ">75.0<" in bars


def test_branching_evidence_reduces_complete_tables_and_refuses_broken_ones():
    from experiments.synbios_moe.mechanisms.comparison_report import branching_evidence
    from experiments.synbios_moe.mechanisms.token_routes import ROUTE_PROTOCOL

    summary = {"protocol": ROUTE_PROTOCOL, "parameters_updated": False, "examples": 30, "attributes": {"university": 10, "major": 20, "company": 0},
               "layers": 2, "experts": 4, "top_k": 2}
    pair_rows, nmi_rows = [], []
    for a, n in (("university", 10), ("major", 30)):
        for layer in (0, 1):
            pair_rows.append({"attribute": a, "layer": str(layer), "pair_group": "same_t2", "pair_count": str(n), "t1_route_overlap": "0.9",
                              "t2_route_overlap": "0.8", "branching_score": "0.1"})
            pair_rows.append({"attribute": a, "layer": str(layer), "pair_group": "different_t2", "pair_count": str(2 * n), "t1_route_overlap": "0.9",
                              "t2_route_overlap": str(0.5 - 0.1 * layer), "branching_score": str(0.4 + 0.1 * layer)})
            nmi_rows.append({"attribute": a, "layer": str(layer), "examples": "5", "t1_top1_token_nmi": str(0.2 + 0.1 * layer), "t2_top1_token_nmi": "0.5"})
    by_layer, detail, head = branching_evidence(summary, pair_rows, nmi_rows)
    assert [r["layer"] for r in by_layer] == [0, 1] and len(detail) == 4
    assert by_layer[0]["same_t2_pair_count"] == 40 and by_layer[0]["different_t2_pair_count"] == 80
    assert by_layer[0]["difference_in_differences"] == pytest.approx(0.3) and by_layer[1]["difference_in_differences"] == pytest.approx(0.4)
    assert head["difference_in_differences"] == pytest.approx(0.35) and head["all_layers_positive"] and head["bad_case_examples"] == 30
    assert head["max_t1_nmi_by_attribute"] == {"university": pytest.approx(0.3), "major": pytest.approx(0.3)}
    with pytest.raises(ValueError, match="not complete"):
        branching_evidence(summary, pair_rows[:-1], nmi_rows)
    broken = [dict(r) for r in pair_rows]
    broken[0]["branching_score"] = "0.3"
    with pytest.raises(ValueError, match="branching score"):
        branching_evidence(summary, broken, nmi_rows)
    with pytest.raises(ValueError, match="do not close"):
        branching_evidence({**summary, "examples": 31}, pair_rows, nmi_rows)
    with pytest.raises(ValueError, match="protocol"):
        branching_evidence({**summary, "protocol": "other"}, pair_rows, nmi_rows)


def test_line_chart_and_the_reports_that_use_it(tmp_path):
    import xml.etree.ElementTree as ET

    from experiments.synbios_moe.mechanisms.company_relation import fit_company_pair, paired_exposure
    from experiments.synbios_moe.pretraining.dataset import WHOLE_ATTRIBUTES
    from experiments.synbios_moe.probes.figures import line_chart_svg

    svg = line_chart_svg({"a": [0.1, 0.5, 0.9], "fit <b>": [0.2, 0.5, 0.8]}, title="t", x_labels=["P0", "P1", "P2"], dashed=("fit <b>",))
    root = ET.fromstring(svg)
    assert len(root.findall("{http://www.w3.org/2000/svg}polyline")) == 2 and svg.count("<circle") == 3 and "stroke-dasharray" in svg
    assert "fit &lt;b&gt;" in svg
    with pytest.raises(ValueError):
        line_chart_svg({"a": [0.1]}, title="t", x_labels=["P0", "P1"])
    x = paired_exposure()
    curves = {a: (0.2 + 0.6 * x if a in ("company", "company_city") else 0.3 + 0.0 * x) for a in WHOLE_ATTRIBUTES}
    out = fit_company_pair(curves, tmp_path / "company")
    assert out["pair_mean_gain"] == pytest.approx(0.6, abs=1e-9)
    figure = (tmp_path / "company" / "company_relation.svg").read_text()
    assert ET.fromstring(figure).tag.endswith("svg") and "partner exposure" in figure and figure.count("<polyline") == 5


def test_ground_truth_first_protocol_audit_on_real_artifacts(studies, tmp_path):
    """The reference script's command line: the protocol is audited on the artifacts a run would use.  The fixture holds the
    original P-whole probe of one attribute only, so that task passes and the other four are reported as not ready."""

    s = studies["single"]
    out = tmp_path / "audit" / "protocol.json"
    done = subprocess.run([sys.executable, str(ROOT / "scripts" / "audit_ground_truth_first_probe.py"), "--data", str(s["data"]), "--probe-cache", str(s["cache"]),
                           "--probe-dir", str(s["probes"]), "--model-config", studies["model_config"], "--checkpoint", studies["checkpoint"],
                           "--device", "cpu", "--codec", "bytes", "--output", str(out)], capture_output=True, text=True, timeout=600)
    assert done.returncode == 1, done.stdout[-1500:] + done.stderr[-2500:]               # four of five tasks have no reference probe yet
    record = json.loads(out.read_text())
    assert record["protocol"] == "ground_truth_first_whole_rank_matched_v1" and not record["quality_gate_passed"] and len(record["tasks"]) == 5
    by_attribute = {t["attribute"]: t for t in record["tasks"]}
    good = by_attribute["university"]
    assert good["passed"] and good["errors"] == [] and good["sampled_items_checked"] >= 12 and good["rank"] == 2
    assert good["trainable_parameters"] == ["delta.a.weight", "delta.b.weight", "normalizer.weight", "normalizer.bias", "classifier.weight", "classifier.bias"]
    assert good["expanded_train_examples"] == 6 * good["train_sources"] and len(good["reference_whole_probe_sha256"]) == 64
    assert all(not by_attribute[a]["passed"] and by_attribute[a]["errors"] for a in ("birth_city", "major", "company", "company_city"))
    # record mode still wants records
    assert subprocess.run([sys.executable, str(ROOT / "scripts" / "audit_ground_truth_first_probe.py")], capture_output=True, text=True).returncode == 2
