"""Documentation hygiene: every repository path that the documentation names exists."""

import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
TOP_LEVEL = ("mini_train_sys_b200/", "experiments/", "scripts/", "configs/", "tests/", "docs/", "examples/", "profiles/")
SUFFIXES = (".py", ".cu", ".cuh", ".cpp", ".h", ".yaml", ".md", ".sh", ".ps1", ".ipynb", ".txt")


def _documents():
    yield from sorted((ROOT / "docs").glob("*.md"))
    for name in ("README.md", "CONTRIBUTING.md", "configs/README.md", "scripts/README.md", "scripts/synbios_moe_runbook.md",
                 "examples/README.md", "profiles/README.md", "experiments/synbios_moe/README.md"):
        yield ROOT / name


def _expand(token: str) -> list[str]:
    """``a/{b,c}.py`` -> ``a/b.py``, ``a/c.py`` (nested groups too)."""

    group = re.search(r"\{([^{}]*)\}", token)
    if group is None:
        return [token]
    return [t for alt in group.group(1).split(",") for t in _expand(token[:group.start()] + alt.strip() + token[group.end():])]


def test_paths_named_in_the_documentation_exist():
    missing = []
    for doc in _documents():
        assert doc.is_file(), doc
        for token in re.findall(r"`([^`\n]+)`", doc.read_text(encoding="utf-8")):
            token = token.split("::")[0].split(":")[0].strip().lstrip("./")
            if not token.startswith(TOP_LEVEL) or not token.endswith(SUFFIXES) or any(ch in token for ch in " <>$%"):
                continue
            for path in _expand(token):
                found = list(ROOT.glob(path)) if "*" in path else [ROOT / path] if (ROOT / path).exists() else []
                if not found:
                    missing.append(f"{doc.relative_to(ROOT)}: {path}")
    assert not missing, missing


def test_docs_index_lists_every_page():
    index = (ROOT / "docs" / "README.md").read_text(encoding="utf-8")
    pages = sorted(p.name for p in (ROOT / "docs").glob("*.md") if p.name != "README.md")
    assert pages and all(f"`{name}`" in index for name in pages), [n for n in pages if f"`{n}`" not in index]
