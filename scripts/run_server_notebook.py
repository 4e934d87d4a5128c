#!/usr/bin/env python
"""Run a walkthrough unattended and keep a per-cell record of what happened.

Accepts a Jupyter notebook (``.ipynb``: its code cells are executed in order in one namespace; no Jupyter packages are
needed, the file is plain JSON) or a Python walkthrough (``.py``: cut into cells at ``# %%`` markers, or run as a single
cell when it has none, with ``__name__ == "__main__"``).  For every cell the runner stores source, captured output, the
traceback of an exception and the wall time in ``<output>.json``; optionally an executed copy of the notebook with the
outputs filled in.  The exit code is non-zero when any cell raised, which is what makes the walkthroughs usable as server
acceptance tests (reference: scripts/run_server_notebook.py:1-125, which drives nbclient).

    python scripts/run_server_notebook.py examples/training_walkthrough.py --output runs/walkthrough.json

``--export-ipynb PATH`` writes the cells of a ``.py`` walkthrough as a Jupyter notebook instead of running them
(``# %% [markdown]`` blocks become markdown cells); ``examples/notebooks/*.ipynb`` are made this way and a test keeps
them equal to their sources.
"""

from __future__ import annotations

import argparse
import contextlib
import io
import json
import sys
import time
import traceback
from pathlib import Path


def load_cells(path: Path) -> list[str]:
    if path.suffix == ".ipynb":
        notebook = json.loads(path.read_text(encoding="utf-8"))
        cells = []
        for cell in notebook.get("cells", []):
            if cell.get("cell_type") == "code":
                src = cell.get("source", "")
                cells.append("".join(src) if isinstance(src, list) else str(src))
        return cells
    text = path.read_text(encoding="utf-8")
    if "\n# %%" not in "\n" + text:
        return [text]
    cells, current = [], []
    for line in text.splitlines(keepends=True):
        if line.startswith("# %%") and current:
            cells.append("".join(current))
            current = []
        current.append(line)
    if current:
        cells.append("".join(current))
    return cells


def percent_cells(text: str) -> list[tuple[str, str]]:
    """(kind, source) for every ``# %%`` cell of a percent-format script; kind is "code" or "markdown".

    Text before the first marker (a shebang, a module docstring) is a code cell of its own when it holds anything but
    blank lines.  A markdown cell's source is its comment lines without the leading ``# ``.
    """

    cells: list[tuple[str, list[str]]] = [("code", [])]
    for line in text.splitlines():
        if line.startswith("# %%"):
            cells.append(("markdown" if "[markdown]" in line else "code", []))
        else:
            cells[-1][1].append(line)
    out = []
    for kind, lines in cells:
        if kind == "markdown":
            lines = [ln[2:] if ln.startswith("# ") else ln.lstrip("#") for ln in lines]
        while lines and not lines[0].strip():
            lines.pop(0)
        while lines and not lines[-1].strip():
            lines.pop()
        if lines and not (kind == "code" and all(ln.startswith("#!") for ln in lines)):
            out.append((kind, "\n".join(lines)))
    return out


def notebook_from_script(text: str) -> dict:
    """The notebook (nbformat 4.5, no outputs) with the cells of a percent-format script."""

    cells = []
    for index, (kind, source) in enumerate(percent_cells(text)):
        cell = {"cell_type": kind, "id": f"cell-{index:03d}", "metadata": {}, "source": source.splitlines(keepends=True)}
        if kind == "code":
            cell.update(execution_count=None, outputs=[])
        cells.append(cell)
    return {"cells": cells, "nbformat": 4, "nbformat_minor": 5,
            "metadata": {"kernelspec": {"display_name": "Python 3", "language": "python", "name": "python3"},
                         "language_info": {"name": "python"}}}


def export_notebook(source: Path, destination: Path) -> int:
    notebook = notebook_from_script(source.read_text(encoding="utf-8"))
    destination.parent.mkdir(parents=True, exist_ok=True)
    destination.write_text(json.dumps(notebook, indent=1, ensure_ascii=False) + "\n", encoding="utf-8")
    return len(notebook["cells"])


def _strip_magics(source: str) -> str:
    """IPython line magics and shell escapes are not Python: comment them out so that the rest of the cell still runs."""

    return "".join(("# " + line) if line.lstrip().startswith(("%", "!")) else line for line in source.splitlines(keepends=True))


class CellTimeout(Exception):
    pass


@contextlib.contextmanager
def _cell_deadline(seconds: float):
    """Raise ``CellTimeout`` inside the cell when it runs longer than ``seconds`` (main thread, POSIX timers; <= 0: no limit)."""

    import signal

    if seconds is None or seconds <= 0 or not hasattr(signal, "setitimer"):
        yield
        return

    def expired(signum, frame):
        raise CellTimeout(f"cell ran longer than {seconds:g} s")

    previous = signal.signal(signal.SIGALRM, expired)
    signal.setitimer(signal.ITIMER_REAL, seconds)
    try:
        yield
    finally:
        signal.setitimer(signal.ITIMER_REAL, 0)
        signal.signal(signal.SIGALRM, previous)


def run_cells(cells: list[str], *, filename: str, keep_going: bool = False, echo: bool = False, timeout_seconds: float = -1) -> list[dict]:
    namespace: dict = {"__name__": "__main__", "__file__": filename}
    records = []
    for index, source in enumerate(cells):
        out, err = io.StringIO(), io.StringIO()
        started = time.perf_counter()
        record = {"cell": index, "source": source, "status": "ok", "error": None}
        try:
            code = compile(_strip_magics(source), f"{filename}#cell{index}", "exec")
            with contextlib.redirect_stdout(out), contextlib.redirect_stderr(err), _cell_deadline(timeout_seconds):
                exec(code, namespace)      # noqa: S102 - executing the user's own walkthrough is the purpose of this tool
        except SystemExit as exc:          # a walkthrough that ends with sys.exit(main())
            if exc.code not in (None, 0):
                record.update(status="error", error=f"SystemExit({exc.code!r})")
        except BaseException:              # noqa: BLE001 - the record is the product; the cell's failure must not kill the runner
            record.update(status="error", error=traceback.format_exc())
        record.update(stdout=out.getvalue(), stderr=err.getvalue(), seconds=round(time.perf_counter() - started, 3))
        records.append(record)
        if echo:
            print(f"[cell {index}] {record['status']} in {record['seconds']} s", flush=True)
        if record["status"] == "error" and not keep_going:
            break
    return records


def write_executed_notebook(source: Path, records: list[dict], destination: Path) -> None:
    notebook = json.loads(source.read_text(encoding="utf-8"))
    by_index = {r["cell"]: r for r in records}
    code_index = 0
    for cell in notebook.get("cells", []):
        if cell.get("cell_type") != "code":
            continue
        rec = by_index.get(code_index)
        code_index += 1
        if rec is None:
            continue
        outputs = []
        if rec["stdout"]:
            outputs.append({"output_type": "stream", "name": "stdout", "text": rec["stdout"]})
        if rec["error"]:
            outputs.append({"output_type": "error", "ename": "Exception", "evalue": rec["error"].strip().splitlines()[-1],
                            "traceback": rec["error"].splitlines()})
        cell["outputs"], cell["execution_count"] = outputs, rec["cell"] + 1
    destination.parent.mkdir(parents=True, exist_ok=True)
    destination.write_text(json.dumps(notebook, indent=1), encoding="utf-8")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("walkthrough", type=Path)
    ap.add_argument("--output", type=Path, help="JSON record (default: <walkthrough>.run.json)")
    ap.add_argument("--executed-notebook", type=Path, help="for .ipynb inputs: write a copy with the outputs filled in")
    ap.add_argument("--export-ipynb", type=Path, help="for .py inputs: write the cells as a notebook and exit without running them")
    ap.add_argument("--keep-going", action="store_true", help="run the remaining cells after a failure")
    ap.add_argument("--output-dir", type=Path, help="write <name>.run.json and, for notebooks, <name>.executed.ipynb into this directory "
                                                    "(the reference's option; --output / --executed-notebook name the files one by one)")
    ap.add_argument("--timeout-seconds", type=float, default=-1, help="limit per cell; -1: none")
    ap.add_argument("--kernel", help="accepted for the reference's command lines: cells run in this process, no Jupyter kernel is started")
    ap.add_argument("--quiet", action="store_true")
    args = ap.parse_args(argv)
    path = args.walkthrough.resolve()
    if args.export_ipynb is not None:
        if path.suffix != ".py":
            ap.error("--export-ipynb wants a .py walkthrough")
        print(json.dumps({"notebook": str(args.export_ipynb), "cells": export_notebook(path, args.export_ipynb)}))
        return 0
    cells = load_cells(path)
    records = run_cells(cells, filename=str(path), keep_going=args.keep_going, echo=not args.quiet, timeout_seconds=args.timeout_seconds)
    failed = [r["cell"] for r in records if r["status"] == "error"]
    report = {"walkthrough": str(path), "cells": len(cells), "executed": len(records), "failed_cells": failed,
              "seconds": round(sum(r["seconds"] for r in records), 3), "records": records}
    if args.output_dir is not None:
        args.output = args.output or args.output_dir / f"{path.stem}.run.json"
        if path.suffix == ".ipynb" and args.executed_notebook is None:
            args.executed_notebook = args.output_dir / f"{path.stem}.executed.ipynb"
    output = args.output or path.with_suffix(".run.json")
    output.parent.mkdir(parents=True, exist_ok=True)
    output.write_text(json.dumps(report, indent=1), encoding="utf-8")
    if args.executed_notebook and path.suffix == ".ipynb":
        write_executed_notebook(path, records, args.executed_notebook)
    if failed and not args.quiet:
        print(records[failed[0]]["error"], file=sys.stderr)
    print(json.dumps({k: report[k] for k in ("cells", "executed", "failed_cells", "seconds")}))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
