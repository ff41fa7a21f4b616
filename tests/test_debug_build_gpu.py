"""The debug build of the kernels (``TORCHLLMS_B200_DEBUG=1``: compiled with ``-DTL_DEBUG``, every
index taken from a step's index data range-checked on the device, and ``Engine.prepare`` checking
the same arrays on the host) gives the release build's logits on sound input and reports nothing.
Only sound input is run: a bad index is what the host check is for (``tests/test_engine_cpu.py``),
and no test feeds a kernel one.  The reference checks its layout on the host
(torchllms/models/paged_kv.py:797-843)."""

import os

import numpy as np
import pytest
import torch

import traces
from helpers import TINY, run_trace, tiny_folder
from test_replay_gpu import requests_for

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name,dtype", [("C", "bfloat16"), ("D", "float32")])
def test_debug_build_agrees_with_the_release_build(tmp_path, monkeypatch, name, dtype):
    store = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = tiny_folder(tmp_path, name, dtype=store)
    reqs = requests_for(name)
    kw = dict(chunks=(2, 5, 24, 96, 150, 260, 40)) if name == "C" else {}
    steps, places, peak = traces.mixed(reqs, **kw)
    release = run_trace(folder, dtype, steps, tmp_path / "release", max_tokens=peak)
    monkeypatch.setenv("TORCHLLMS_B200_DEBUG", "1")
    debug = run_trace(folder, dtype, steps, tmp_path / "debug", max_tokens=peak, timeout=1800)
    assert set(debug) == set(release) == set(places)
    for step in places:
        assert np.isfinite(debug[step]).all()
        # the same kernels with checks compiled in; decode steps run eagerly instead of from recorded graphs
        np.testing.assert_allclose(debug[step], release[step], rtol=0, atol=1e-5)


def test_debug_libraries_are_built_apart_and_export_the_debug_word(monkeypatch):
    import importlib
    import subprocess
    import sys
    code = ("import os; os.environ['TORCHLLMS_B200_DEBUG']='1';"
            "from torchllms_b200.kernels import build;"
            "p = build.compile_library('rope'); print(p);"
            "lib = build.load_library('rope'); print(lib.tl_debug_take())")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600,
                         cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert out.returncode == 0, out.stderr[-2000:]
    path, word = out.stdout.strip().splitlines()[-2:]
    from torchllms_b200.kernels.build import library_path
    assert path != str(library_path("rope")) and word == "0"
