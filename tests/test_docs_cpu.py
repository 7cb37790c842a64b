"""The guides stay in step with the code: every environment variable the sources read is described in
docs/environment_variables.md, every metric the dashboard shows exists, and the API reference names what the packages export."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _sources(exts):
    for top in ("memfabric_hybrid_b200", "bench.py"):
        path = os.path.join(ROOT, top)
        if os.path.isfile(path):
            yield path
            continue
        for d, _, files in os.walk(path):
            if "__pycache__" in d:
                continue
            for f in files:
                if f.endswith(exts):
                    yield os.path.join(d, f)


def test_every_environment_variable_is_documented():
    doc = open(os.path.join(ROOT, "docs", "environment_variables.md")).read()
    names = set()
    for path in _sources((".cpp", ".h", ".cu", ".cuh")):
        text = open(path, errors="replace").read()
        for m in re.finditer(r'Env(?:Int|Str)\(\s*"([A-Z0-9_]+)"(?:\s*,\s*"([A-Z0-9_]+)")?', text):
            names.update(n for n in m.groups() if n)
        names.update(re.findall(r'getenv\("((?:MF|ZBAL)_[A-Z0-9_]+)"\)', text))
    for path in _sources((".py",)):
        text = open(path, errors="replace").read()
        names.update(re.findall(r'environ(?:\.get|\.setdefault|\.pop)?[\(\[]\s*"((?:MF|ZBAL)_[A-Z0-9_]+)"', text))
    names -= {"ZBAL_OP_DEFUALT_STREAM"}          # a misspelling of the reference that is still honoured, on purpose not advertised
    assert len(names) > 40
    missing = sorted(n for n in names if f"`{n}`" not in doc)
    assert not missing, f"not described in docs/environment_variables.md: {missing}"


def test_api_reference_names_the_exports():
    ref = open(os.path.join(ROOT, "docs", "python_api.md")).read()
    import tensor_rtl
    import zbal
    from memfabric_hybrid_b200 import api
    from memfabric_hybrid_b200.zbal import module as zm
    for name in [n for n in api.__all__ if callable(getattr(api, n, None))] + [n for n in zbal.__all__ if callable(getattr(zm, n, None))] + ["PTensor", "PTensorSet", "BatchP2PExecutor", "MemoryFabricExecutor",
                                                                                  "balanced_placement", "TrainToInferResharder", "BufferPool"]:
        assert f"`{name}" in ref, name
    assert tensor_rtl.PTensor is not None
