"""Concurrent in-tree builds: several processes that find an artefact stale at once must not corrupt it."""
import multiprocessing as mp
import os
import time
from pathlib import Path

from opaque_b200.utils import build


def _writer(target: str, delay: float, marker: str) -> None:
    tgt = Path(target)
    with build._build_lock(tgt):
        if tgt.exists():
            return                       # another process built it while this one waited on the lock
        tmp = tgt.with_suffix(f".tmp{os.getpid()}")
        tmp.write_text(marker[:1])
        time.sleep(delay)                # a slow compile: a second writer must not interleave
        tmp.write_text(marker)
        os.replace(tmp, tgt)


def test_build_lock_serialises_writers(tmp_path):
    target = tmp_path / "artefact.so"
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_writer, args=(str(target), 0.3, f"built-by-{i}" * 50)) for i in range(4)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
        assert p.exitcode == 0
    text = target.read_text()
    assert any(text == f"built-by-{i}" * 50 for i in range(4))      # one complete artefact, from exactly one writer
    assert not list(tmp_path.glob("*.tmp*"))
