"""The programs under examples/ run to completion on CPU."""
import contextlib
import io
import os
import runpy
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("name", ["autograd_demo", "mixed_precision_demo", "profiler_tensorboard_demo", "model_formats_demo",
                                  "distributed_training_demo", "transformer_demo"])
def test_example_runs(name):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"):
        env.pop(k, None)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "examples", name + ".py")], capture_output=True, text=True, timeout=300, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    assert r.stdout.strip()


@pytest.mark.parametrize("name", ["mlp_training", "cnn_demo", "readme_basic_usage_demo", "tensor_nd_demo", "broadcasting_demo",
                                  "activation_demo", "special_functions_demo", "complex_tensor_demo", "fft_demo",
                                  "matrix_decomposition_demo", "linear_regression", "boston_housing_regression", "embedding_demo",
                                  "batchnorm_demo", "adamw_scheduler_demo", "gradient_flow_demo", "neural_network_demo",
                                  "complete_training_demo", "rnn_sequence_demo", "data_loading_demo", "vision_pipeline_demo",
                                  "visualization_demo", "distributions_demo", "quantization_sparsity_demo", "model_hub_demo",
                                  "validation_debug_demo", "llm_decode_demo", "finetune_export_serve_demo", "chat_prompt_demo", "gpu_kernel_demo"])
def test_example_runs_in_process(name, monkeypatch):
    """The single-process examples, run inside this interpreter (no second import of torch per program)."""
    if torch.cuda.is_available():
        pytest.skip("the in-process form is the CPU check; on a GPU box run the programs themselves")
    monkeypatch.syspath_prepend(os.path.join(ROOT, "examples"))
    out = io.StringIO()
    with contextlib.redirect_stdout(out):
        try:
            runpy.run_path(os.path.join(ROOT, "examples", name + ".py"), run_name="__main__")
        except SystemExit as e:
            assert not e.code
    assert out.getvalue().strip()


def test_quickstart_notebook_cells_run(monkeypatch):
    import json
    nb = json.load(open(os.path.join(ROOT, "notebooks", "quickstart.ipynb")))
    assert nb["nbformat"] == 4
    monkeypatch.chdir(os.path.join(ROOT, "notebooks"))
    ns: dict = {}
    out = io.StringIO()
    with contextlib.redirect_stdout(out):
        for cell in nb["cells"]:
            if cell["cell_type"] == "code":
                src = "".join(cell["source"])
                if "IPython" in src and "IPython" not in sys.modules:
                    try:
                        import IPython  # noqa: F401
                    except ImportError:
                        continue
                exec(compile(src, "<notebook cell>", "exec"), ns)
    text = out.getvalue()
    assert "dy/dx = [7.0, 9.0]" in text and "Total params" in text and "epochs" in text


def test_names_imported_in_the_guides_exist():
    """Every ``import`` line inside a Python block of the guides under ``docs/`` and of the README resolves."""
    import glob
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    lines = []
    for path in glob.glob(os.path.join(root, "docs", "*.md")) + [os.path.join(root, "README.md")]:
        text = open(path, encoding="utf-8").read()
        for block in re.findall(r"```python\n(.*?)```", text, flags=re.S):
            lines += [(path, ln.strip()) for ln in block.splitlines() if re.match(r"\s*(from\s+(rustorch|rustorch_b200)[\w.]*\s+import|import\s+(rustorch|rustorch_b200))", ln)]
    assert len(lines) >= 6
    for path, ln in lines:
        try:
            exec(ln, {})
        except Exception as e:  # noqa: BLE001
            raise AssertionError(f"{os.path.basename(path)}: `{ln}` fails: {e}") from None
