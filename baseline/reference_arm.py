"""Reference arm of ``bench.py``: runs the UNMODIFIED reference package installed under
``baseline/_ref`` through its own ``create_train_task`` / ``fsdp2_trainer`` code path on the
same model, data shapes and metric, or reports why it cannot."""
from __future__ import annotations

import json
import os


def _emit(obj) -> None:
    """Result line on the descriptor that ``bench.py`` kept for it (its original stdout)."""
    os.write(int(os.environ.get("BENCH_JSON_FD", "1")), (json.dumps(obj) + "\n").encode())

HERE = os.path.dirname(os.path.abspath(__file__))


def unavailable(reason: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        _emit({"impl": "reference", "unavailable": reason})


def run(args) -> None:
    ref = os.path.join(HERE, "_ref", "lmms_engine")
    if not os.path.isdir(ref):
        unavailable("reference package is not installed under baseline/_ref")
        return
    try:
        from . import reference_run

        reference_run.main(args)
    except BaseException as e:  # the arm must always answer with one JSON line and exit 0
        import traceback

        traceback.print_exc()
        unavailable(f"reference run failed: {type(e).__name__}: {str(e)[:300]}")
