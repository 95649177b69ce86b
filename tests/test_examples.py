"""The example scripts named by the profiles' command lines exist, compile and keep their command-line flags."""
import ast
import pathlib
import re

import pytest

ROOT = pathlib.Path(__file__).resolve().parents[1]
EXAMPLES = sorted((ROOT / "inferrous_b200" / "examples").glob("[a-z]*.py"))


@pytest.mark.parametrize("path", EXAMPLES, ids=lambda p: p.stem)
def test_example_compiles(path):
    compile(path.read_text(), str(path), "exec")


def flags_of(path):
    """Option strings of every add_argument call in the script."""
    found = set()
    for node in ast.walk(ast.parse(path.read_text())):
        if isinstance(node, ast.Call) and getattr(node.func, "attr", "") == "add_argument":
            found.update(a.value for a in node.args if isinstance(a, ast.Constant) and isinstance(a.value, str))
    return found


def test_profile_command_lines_name_existing_examples_and_flags():
    """Every `python -m inferrous_b200.examples.X --flag ...` line in profiles/ runs a committed script with flags it has."""
    pattern = re.compile(r"python -m inferrous_b200\.examples\.(\w+)((?:\s+--?[\w-]+(?:[ =][^\s-][^\s]*)?)*)")
    checked = 0
    for doc in sorted((ROOT / "profiles").glob("*.md")):
        for name, tail in pattern.findall(doc.read_text()):
            script = ROOT / "inferrous_b200" / "examples" / f"{name}.py"
            assert script.exists(), f"{doc.name}: {name}.py is not in the examples"
            known = flags_of(script)
            for flag in re.findall(r"(--[\w-]+)", tail):
                assert flag in known, f"{doc.name}: {name}.py has no {flag}"
            checked += 1
    assert checked >= 5


def test_profile_command_lines_use_flags_bench_has():
    known = flags_of(ROOT / "bench.py")
    checked = 0
    for doc in sorted((ROOT / "profiles").glob("*.md")):
        for line in doc.read_text().splitlines():
            if "python bench.py" not in line:
                continue
            command = line.split("python bench.py", 1)[1].split("#", 1)[0]
            for flag in re.findall(r"(--[\w-]+)", command):
                assert flag in known, f"{doc.name}: bench.py has no {flag}"
            checked += 1
    assert checked >= 5
