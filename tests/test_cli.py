"""The command line: option parsing and the random-model command without a GPU; generation on one."""

import json
import os
import subprocess
import sys

import pytest

from tiny_configs import TINY_A

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_cli(*argv, **kw):
    return subprocess.run([sys.executable, "-m", "omniserver_b200.cli", *argv], cwd=ROOT, capture_output=True, text=True, **kw)


def test_parser_has_the_reference_option_names():
    from omniserver_b200.cli import build_parser
    a = build_parser().parse_args(["generate", "--model", "m", "--prompt-ids", "1,2,3", "--max-running", "4",
                                   "--requests", "6", "--trials", "2", "--out", "o.json", "--temperature", "0.8"])
    assert (a.max_running, a.requests, a.trials, a.out, a.temperature) == (4, 6, 2, "o.json", 0.8)
    assert a.max_prefill_tokens == 8192 and a.max_prefill_per_step == 1 and a.max_seq_len == 4096   # scheduler.py:20-25
    assert a.max_new_tokens == 128                                                                   # request.py:29


def test_random_model_command_writes_a_loadable_folder(tmp_path):
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    p = run_cli("random-model", "--config", str(cfg), "--seed", "3", "--out", str(tmp_path / "m"), "--store-dtype", "float32")
    assert p.returncode == 0, p.stderr
    from safetensors import safe_open
    with safe_open(str(tmp_path / "m" / "model.safetensors"), framework="pt") as f:
        names = set(f.keys())
    assert "model.layers.1.self_attn.k_proj.bias" in names and "lm_head.weight" not in names
    assert json.loads((tmp_path / "m" / "config.json").read_text())["hidden_size"] == 64


@pytest.mark.gpu
def test_generate_command(tmp_path):
    import torch
    from helpers import make_model_dir, plain_model
    from plain import model as pm
    d = make_model_dir(tmp_path, "tiny_a", "float32")
    cfg, w = plain_model(d)
    out = tmp_path / "out.json"
    p = run_cli("generate", "--model", d, "--dtype", "float32", "--prompt-ids", "5,17,3,200,9", "--prompt-ids", "7,7,8",
                "--max-new-tokens", "6", "--max-running", "2", "--max-prefill-per-step", "2", "--out", str(out), timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    res = json.loads(out.read_text())
    assert res["outputs"][0] == pm.generate(cfg, w, [5, 17, 3, 200, 9], 6)
    assert res["outputs"][1] == pm.generate(cfg, w, [7, 7, 8], 6)
    assert "tok/s" in p.stdout
