"""vLLM's own engine with this package as its platform plugin (GPU only).

The plugin is discovered the way vLLM discovers installed plugins: through entry-point
metadata.  The test writes that metadata (what ``pip install`` of this package would put into
site-packages) into a temporary directory on ``PYTHONPATH`` of a child process."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

ENTRY_POINTS = """[vllm.platform_plugins]
b200 = vllm_gcu_b200:register_platform_plugins

[vllm.general_plugins]
b200_models = vllm_gcu_b200:register_custom_models
"""


def _run_worker(tmp_path, check: str):
    info = tmp_path / "vllm_gcu_b200-0.1.0.dist-info"
    info.mkdir()
    (info / "METADATA").write_text("Metadata-Version: 2.1\nName: vllm-gcu-b200\nVersion: 0.1.0\n")
    (info / "entry_points.txt").write_text(ENTRY_POINTS)
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(tmp_path), ROOT, env.get("PYTHONPATH", "")])
    env.pop("VLLM_PLUGINS", None)
    env["B200_PLUGIN_CHECK"] = check
    res = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "_vllm_plugin_worker.py")],
                         env=env, capture_output=True, text=True, timeout=850)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-5000:]
    return res.stdout


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
@pytest.mark.timeout(900)
def test_vllm_engine_runs_on_the_plugin(tmp_path):
    pytest.importorskip("vllm")
    assert "vllm plugin ok" in _run_worker(tmp_path, "base")


@pytest.mark.skipif(not torch.cuda.is_available(), reason="needs a GPU")
@pytest.mark.timeout(900)
def test_vllm_fp8_engine_runs_on_the_plugin_kernels(tmp_path):
    """``quantization="fp8"`` under vLLM: the linear layers select this package's fp8 kernel."""
    pytest.importorskip("vllm")
    assert "vllm fp8 ok" in _run_worker(tmp_path, "fp8")
