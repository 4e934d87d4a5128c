"""Lineage audit of the study: every derived artifact must point at the inputs it was made from.

Three levels (reference: experiments/synbios_moe/audit.py:28-289):

* ``audit_dataset`` / ``dataset_lineage``  raw files against the dataset manifest (size and sha256); the token shards against
  their own manifest and against the dataset (one training document per biography, no held-out language-model split); the
  probe cache against the dataset manifest it embeds, its array hashes and its class coverage.  ``dataset_lineage`` writes
  ``lineage.json`` beside the dataset, the shards and the cache, so that a copied directory still names its parent.
* ``audit_study``  one condition: dataset, cache and a probe pipeline root (results carry an identity, sit beside their
  weights, all jobs finished, all heads trained against the same backbone file).
* ``build_study_audit``  both conditions of the comparison: identical people, matched probe hyper-parameters, exported
  ``model.pt`` hashes recorded; emits ``dataset_lineage.json`` and ``summary.json`` with the list of checks that passed.
"""

from __future__ import annotations

from pathlib import Path

from experiments.synbios_moe.artifact_io import read_json, sha256_file, write_json
from experiments.synbios_moe.probes.dataset import validate_probe_cache

EXPECTED_VARIANT = {"single": "single", "multi5_permute": "multi5+permute"}


def audit_dataset(data_root: str | Path) -> list[str]:
    root = Path(data_root)
    problems = []
    try:
        manifest = read_json(root / "manifest.json")
    except (OSError, ValueError) as exc:
        return [f"{root}: manifest unreadable ({exc})"]
    for name, meta in manifest.get("files", {}).items():
        path = root / name
        if not path.is_file():
            problems.append(f"{root}: {name} missing")
        elif path.stat().st_size != int(meta.get("bytes", path.stat().st_size)) or sha256_file(path) != meta["sha256"]:
            problems.append(f"{root}: {name} differs from the manifest")
    return problems


def _file_record(path: Path, base: Path) -> dict:
    return {"path": str(path.relative_to(base)), "bytes": path.stat().st_size, "sha256": sha256_file(path)}


def _check_manifest_file(root: Path, record: dict, problems: list[str]) -> None:
    path = root / record["path"]
    if not path.is_file():
        problems.append(f"{root}: {record['path']} missing")
    elif path.stat().st_size != int(record["num_bytes"]) or sha256_file(path) != record["sha256"]:
        problems.append(f"{root}: {record['path']} differs from the shard manifest")


def audit_token_shards(token_root: str | Path, data_manifest: dict | None = None) -> list[str]:
    root = Path(token_root)
    try:
        manifest = read_json(root / "manifest.json")
    except (OSError, ValueError) as exc:
        return [f"{root}: shard manifest unreadable ({exc})"]
    problems: list[str] = []
    train, held = manifest["splits"]["train"], manifest["splits"]["validation"]
    if data_manifest is not None and int(train["documents"]) != int(data_manifest.get("num_biographies", -1)):
        problems.append(f"{root}: {train['documents']} training documents for {data_manifest.get('num_biographies')} biographies")
    if int(held["documents"]) != 0:
        problems.append(f"{root}: the pre-training shards have a held-out split ({held['documents']} documents)")
    for shard in [*train["shards"], *held["shards"]]:
        _check_manifest_file(root, shard, problems)
    for split in (train, held):
        _check_manifest_file(root, split["document_index"], problems)
    if sum(int(s["num_tokens"]) for s in train["shards"]) != int(train["tokens"]):
        problems.append(f"{root}: shard token counts do not add up to the split total")
    return problems


def dataset_lineage(condition: str, data_root: str | Path, probe_cache: str | Path, *, token_root: str | Path | None = None,
                    write: bool = True) -> dict:
    """Verify dataset -> token shards -> probe cache of one condition and describe the chain; raises on any mismatch."""

    data_root, cache_root = Path(data_root), Path(probe_cache)
    token_root = Path(token_root) if token_root is not None else data_root / "token_shards"
    problems = audit_dataset(data_root)
    data_manifest = read_json(data_root / "manifest.json")
    if condition in EXPECTED_VARIANT and data_manifest.get("variant") != EXPECTED_VARIANT[condition]:
        problems.append(f"{data_root}: variant {data_manifest.get('variant')!r} is not the {condition} corpus")
    problems += audit_token_shards(token_root, data_manifest)
    cache_manifest = read_json(cache_root / "manifest.json")
    if cache_manifest.get("source_manifest") != data_manifest:
        problems.append(f"{cache_root}: the cache embeds a different dataset manifest")
    verdict = validate_probe_cache(cache_root, data_root)
    problems += [f"{cache_root}: {e}" for e in verdict["errors"]]
    uncovered = {k: c["validation_only_classes"] for k, c in cache_manifest.get("coverage", {}).items() if c["validation_only_classes"]}
    if problems:
        raise ValueError("; ".join(problems))
    parent = sha256_file(data_root / "manifest.json")
    token_manifest = read_json(token_root / "manifest.json")
    lineage = {
        "format_version": 1, "condition": condition,
        "source_dataset": {"path": str(data_root.resolve()), "manifest_sha256": parent,
                           "profiles_sha256": data_manifest["files"]["profiles.jsonl"]["sha256"],
                           "people": int(data_manifest["num_people"]), "biographies": int(data_manifest["num_biographies"])},
        "token_shards": {"path": str(token_root.resolve()), "manifest_sha256": sha256_file(token_root / "manifest.json"),
                         "parent_manifest_sha256": parent, "documents": int(token_manifest["splits"]["train"]["documents"]),
                         "tokens": int(token_manifest["splits"]["train"]["tokens"]),
                         "split_semantics": "every generated biography is a pre-training document; nothing is held out",
                         "files": [_file_record(p, token_root) for p in sorted(token_root.rglob("*")) if p.is_file() and p.name != "lineage.json"]},
        "probe_cache": {"path": str(cache_root.resolve()), "manifest_sha256": sha256_file(cache_root / "manifest.json"),
                        "parent_manifest_sha256": parent, "profiles": int(cache_manifest["profiles"]),
                        "p_examples": int(cache_manifest["p_examples"]), "q_examples": int(cache_manifest["q_examples"]),
                        "split_semantics": "person-level probe train / validation split; pre-training saw both parts",
                        "validation_only_classes": uncovered,
                        "files": [_file_record(p, cache_root) for p in sorted(cache_root.iterdir()) if p.is_file() and p.name != "lineage.json"]},
    }
    if write:
        write_json(data_root / "lineage.json", lineage)
        write_json(token_root / "lineage.json", {"format_version": 1, "condition": condition, **lineage["token_shards"]})
        write_json(cache_root / "lineage.json", {"format_version": 1, "condition": condition, **lineage["probe_cache"]})
    return lineage


def audit_pipeline(pipeline_root: str | Path) -> list[str]:
    root = Path(pipeline_root)
    problems: list[str] = []
    backbones = set()
    for path in sorted((root / "training").glob("*.json")):
        rec = read_json(path)
        if "identity" not in rec:
            problems.append(f"{path}: result without identity")
        else:
            backbones.add(rec["identity"].get("checkpoint_model_sha256"))
        if not path.with_suffix(".pt").is_file():
            problems.append(f"{path}: weights missing beside the result")
    if len(backbones - {None}) > 1:
        problems.append(f"{root}: heads were trained against {len(backbones - {None})} different backbone files")
    state = root / "pipeline.json"
    if state.is_file():
        data = read_json(state)
        unfinished = [n for n, j in data.get("jobs", {}).items() if j.get("status") not in ("done", "skipped")]
        if unfinished:
            problems.append(f"{state}: unfinished jobs {unfinished[:5]}{'...' if len(unfinished) > 5 else ''}")
    return problems


def audit_study(*, data_root: str | Path | None = None, probe_cache: str | Path | None = None,
                pipeline_root: str | Path | None = None) -> dict:
    problems: list[str] = []
    if data_root is not None:
        problems += audit_dataset(data_root)
        if (Path(data_root) / "token_shards" / "manifest.json").is_file():
            problems += audit_token_shards(Path(data_root) / "token_shards", read_json(Path(data_root) / "manifest.json"))
    if probe_cache is not None:
        verdict = validate_probe_cache(probe_cache, data_root)
        problems += [f"{probe_cache}: {e}" for e in verdict["errors"]]
    if pipeline_root is not None:
        problems += audit_pipeline(pipeline_root)
    return {"ok": not problems, "problems": problems}


def build_study_audit(conditions: dict[str, dict], output_dir: str | Path) -> dict:
    """``conditions``: ``{"single": {...}, "multi5_permute": {...}}`` with ``data``, ``probe_cache`` and optionally
    ``pipeline`` (formal probe root) and ``model`` (exported ``model.pt``).  Raises on the first broken link."""

    if set(conditions) != set(EXPECTED_VARIANT):
        raise ValueError(f"expected exactly the conditions {sorted(EXPECTED_VARIANT)}")
    checks = ["raw_dataset_file_sizes_and_hashes", "token_shard_file_sizes_and_hashes", "one_training_document_per_biography",
              "probe_cache_schema_shapes_offsets_and_hashes", "dataset_cache_parent_lineage"]
    lineages = {c: dataset_lineage(c, spec["data"], spec["probe_cache"], token_root=spec.get("token_shards")) for c, spec in conditions.items()}
    if lineages["single"]["source_dataset"]["profiles_sha256"] != lineages["multi5_permute"]["source_dataset"]["profiles_sha256"]:
        raise ValueError("single and multi5_permute do not describe the same people")
    checks.append("identical_profiles_across_conditions")
    records: dict[str, dict] = {}
    for condition, spec in conditions.items():
        rec = {"data_manifest_sha256": lineages[condition]["source_dataset"]["manifest_sha256"],
               "probe_cache_manifest_sha256": lineages[condition]["probe_cache"]["manifest_sha256"]}
        if spec.get("model"):
            rec["model_sha256"] = sha256_file(spec["model"])
        if spec.get("pipeline"):
            problems = audit_pipeline(spec["pipeline"])
            if problems:
                raise ValueError("; ".join(problems))
        records[condition] = rec
    if all(spec.get("pipeline") for spec in conditions.values()):
        from experiments.synbios_moe.probes.comparison_report import load_formal_run, validate_matched_runs

        runs = [load_formal_run(c, conditions[c]["pipeline"], conditions[c]["probe_cache"]) for c in ("single", "multi5_permute")]
        validate_matched_runs(*runs)
        checks += ["probe_results_complete_with_weights", "matched_single_multi_probe_hyperparameters"]
    out = Path(output_dir)
    out.mkdir(parents=True, exist_ok=True)
    write_json(out / "dataset_lineage.json", lineages)
    summary = {"status": "passed", "format_version": 1, "checks": checks, "conditions": records,
               "catalogs": {"dataset_lineage": "dataset_lineage.json"}}
    write_json(out / "summary.json", summary)
    return summary
