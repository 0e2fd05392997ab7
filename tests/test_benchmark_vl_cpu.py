"""The vision-language benchmark builds and serves a tiny random model of every family."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _load():
    path = os.path.join(ROOT, "benchmarks", "benchmark_vision_language.py")
    spec = importlib.util.spec_from_file_location("bench_vl", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.timeout(300)
@pytest.mark.parametrize("family,image_tokens", [
    ("qwen2_5_vl", 6), ("qwen2_vl", 6), ("glm4v", 6), ("llava", 16), ("llava_next", 88), ("internvl", 12),
    ("deepseek_vl2", 17)])
def test_every_family_runs(family, image_tokens):
    res = _load().main(["--family", family, "--device", "cpu", "--layers", "2", "--hidden", "128",
                        "--vision-layers", "2", "--vision-hidden", "128", "--image-size", "56",
                        "--grid", "6", "4", "--tiles", "3", "--num-prompts", "2",
                        "--output-len", "2", "--text-len", "8", "--dtype", "float32",
                        "--vocab", "1000", "--max-model-len", "512"])
    assert res["image_tokens_per_request"] == image_tokens
    assert res["output_tokens_per_s"] > 0
