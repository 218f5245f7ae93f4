"""Every ``torch.load`` in the package passes ``weights_only=True`` (AST scan), and a pickle payload
with a ``__reduce__`` side effect is refused by the checkpoint loader."""
import ast
import pickle
from pathlib import Path

import pytest
import torch

PKG = Path(__file__).resolve().parent.parent / "solarwm_b200"


def test_every_torch_load_is_weights_only():
    offenders = []
    for path in PKG.rglob("*.py"):
        tree = ast.parse(path.read_text())
        for node in ast.walk(tree):
            if isinstance(node, ast.Call) and isinstance(node.func, ast.Attribute) and node.func.attr == "load" \
                    and isinstance(node.func.value, ast.Name) and node.func.value.id == "torch":
                kw = {k.arg: k.value for k in node.keywords}
                ok = "weights_only" in kw and isinstance(kw["weights_only"], ast.Constant) and kw["weights_only"].value is True
                if not ok:
                    offenders.append(f"{path.relative_to(PKG)}:{node.lineno}")
    assert not offenders, offenders


class _Boom:
    def __reduce__(self):
        return (Path("/tmp/_solar_pwned").write_text, ("x",))


def test_pickle_payload_is_not_executed(tmp_path):
    Path("/tmp/_solar_pwned").unlink(missing_ok=True)
    f = tmp_path / "model.pt"
    f.write_bytes(pickle.dumps({"generator": _Boom()}))
    with pytest.raises(Exception):
        torch.load(f, map_location="cpu", weights_only=True)
    assert not Path("/tmp/_solar_pwned").exists()
