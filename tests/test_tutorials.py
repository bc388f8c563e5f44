"""Every tutorial notebook's code cells run top to bottom on CPU (their own assertions included)."""
import ast
import json
from pathlib import Path

import pytest

TUTORIALS = sorted((Path(__file__).resolve().parent.parent / "docs" / "tutorials").glob("*.ipynb"))


@pytest.mark.parametrize("path", TUTORIALS, ids=lambda p: p.stem)
def test_tutorial_runs(path, monkeypatch, tmp_path):
    monkeypatch.chdir(tmp_path)
    nb = json.loads(path.read_text())
    ns = {"__name__": "__tutorial__"}
    ran = 0
    for cell in nb["cells"]:
        if cell["cell_type"] != "code":
            continue
        code = "".join(cell["source"])
        exec(compile(ast.parse(code), f"{path.name}[{ran}]", "exec"), ns)
        ran += 1
    assert ran >= 1
