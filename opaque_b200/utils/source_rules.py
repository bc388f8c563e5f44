"""Static rules for the CUDA sources of this package, checked without a GPU (``python -m opaque_b200.utils.source_rules``).

The kernels run on shared multi-GPU machines where a hang or a fault costs other users their GPU, so a few properties
are enforced on the text of the sources rather than left to review:

1. ``raw-mbarrier-wait`` — the ``mbarrier.try_wait`` / ``test_wait`` instructions appear only inside the single-try helper
   of ``common.cuh``; every caller loops through a helper that counts its tries, records a status code when the budget
   runs out and returns, so no kernel can wait on a barrier forever.
2. ``multicast-load`` — no bulk / tensor copy carries the cluster-multicast qualifier (such a load from another GPU's memory hangs
   the device); ``tcgen05.commit`` may multicast its barrier arrival.
3. ``device-trap`` — no ``__trap()``, ``asm("trap")`` or device ``assert``: a kernel reports through its status word and
   returns, the context stays usable.
4. ``batched-copy-api`` — the batched asynchronous memcpy entry points of the runtime and the driver are not named
   anywhere (they fault on the driver this package is deployed with).
5. ``unbounded-spin`` — a ``while`` / ``for`` loop whose condition or body polls memory (``volatile`` reads, ``ld.acquire``,
   ``ld.relaxed``) must mention a counter or a clock (``tries``, ``spins``, ``budget``, ``clock``, ``globaltimer``, ``limit``).

Parity: the reference has no device code of its own; this takes the place of its sanitizer lanes
(.github/workflows/rust-tests.yml, packages/opaque-accounting sanitizer jobs) for the CUDA side.
"""
from __future__ import annotations

import os
import re
import sys
from dataclasses import dataclass

CUDA_SUFFIXES = (".cu", ".cuh", ".h", ".hpp", ".cpp")
ALL_SUFFIXES = CUDA_SUFFIXES + (".py",)

_BATCHED = re.compile(r"cu(?:da)?Memcpy(?:3D)?Batch" + "Async")
_RAW_WAIT = re.compile(r"mbarrier\.(?:try_wait|test_wait)")
_MULTICAST = re.compile("multicast" + "::" + "cluster")
_TRAP = re.compile(r"__trap\s*\(|\bassert\s*\(|asm[^;]*\"\s*trap\s*;")
_LOOP = re.compile(r"^\s*(?:while\s*\(|for\s*\(|do\s*\{)")
_POLL = re.compile(r"volatile|ld\.acquire|ld\.relaxed|ld\.global\.acquire")
_BOUND = re.compile(r"tries|spins|budget|clock|globaltimer|limit|deadline|iter", re.I)


@dataclass(frozen=True)
class Finding:
    rule: str
    path: str
    line: int
    text: str

    def __str__(self) -> str:
        return f"{self.path}:{self.line}: [{self.rule}] {self.text.strip()[:160]}"


def _strip_comment(line: str) -> str:
    i = line.find("//")
    return line if i < 0 else line[:i]


def check_text(path: str, text: str) -> list[Finding]:
    """Findings for one file's text (``path`` only decides which rules apply and labels the findings)."""
    out: list[Finding] = []
    lines = text.splitlines()
    cuda = path.endswith(CUDA_SUFFIXES)
    in_helper = False
    for n, raw in enumerate(lines, start=1):
        if _BATCHED.search(raw):
            out.append(Finding("batched-copy-api", path, n, raw))
        if not cuda:
            continue
        code = _strip_comment(raw)
        if "bool mbar_try_wait(" in code:
            in_helper = True
        if _RAW_WAIT.search(code) and not (in_helper and os.path.basename(path) == "common.cuh"):
            out.append(Finding("raw-mbarrier-wait", path, n, raw))
        if in_helper and code.startswith("}"):
            in_helper = False
        if _MULTICAST.search(code) and "tcgen05.commit" not in code:
            out.append(Finding("multicast-load", path, n, raw))
        if _TRAP.search(code) and "static_assert" not in code:
            out.append(Finding("device-trap", path, n, raw))
        if _LOOP.match(code):
            # the loop's text: up to the line that closes its first brace (or 12 lines for brace-less forms)
            depth, body = 0, []
            for m in range(n - 1, min(len(lines), n + 40)):
                seg = _strip_comment(lines[m])
                body.append(seg)
                depth += seg.count("{") - seg.count("}")
                if depth <= 0 and m > n - 1:
                    break
                if depth <= 0 and "{" not in seg and seg.rstrip().endswith(";"):
                    break
            blob = "\n".join(body)
            if _POLL.search(blob) and not _BOUND.search(blob):
                out.append(Finding("unbounded-spin", path, n, raw))
    return out


def check_tree(root: str, *, skip: tuple[str, ...] = ("_work", "gpurun_out", ".git", "baseline/_ref", "__pycache__", "build")) -> list[Finding]:
    """Findings for every source file below ``root`` (this module's own patterns are exempt)."""
    found: list[Finding] = []
    me = os.path.abspath(__file__)
    for base, dirs, files in os.walk(root):
        rel = os.path.relpath(base, root)
        dirs[:] = [d for d in dirs if not any((os.path.join(rel, d) if rel != "." else d).startswith(s) for s in skip)]
        for f in sorted(files):
            p = os.path.join(base, f)
            if not f.endswith(ALL_SUFFIXES) or os.path.abspath(p) == me:
                continue
            try:
                text = open(p, encoding="utf-8", errors="replace").read()
            except OSError:
                continue
            found.extend(check_text(os.path.relpath(p, root), text))
    return found


def main(argv: list[str] | None = None) -> int:
    """Command line: check the tree at ``argv[0]`` (default: this repository), print the findings, return 1 if there are any."""
    args = list(sys.argv[1:] if argv is None else argv)
    root = args[0] if args else os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    found = check_tree(root)
    for f in found:
        print(f)
    print(f"{len(found)} finding(s) in {root}")
    return 1 if found else 0


if __name__ == "__main__":
    sys.exit(main())
