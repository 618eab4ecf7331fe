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


def test_bench_subcommands_parse_and_the_byte_and_flop_counts_are_the_tables():
    """The bench sub-commands of the command line, and the counts that the roofline fractions rest on: bytes of a
    decode step and flops of a prompt for the three sizes of the architecture."""
    from omniserver_b200 import benchmark as bm
    from omniserver_b200.cli import build_parser
    a = build_parser().parse_args(["bench", "mixed", "--model", "7b", "--requests", "64", "--max-running", "64", "--chunk", "2048"])
    assert (a.what, a.model, a.requests, a.chunk, a.prompt_lo, a.prompt_hi, a.max_new_tokens) == ("mixed", "7b", 64, 2048, 128, 4096, 256)
    a = build_parser().parse_args(["bench", "decode", "--batch", "64", "--profile"])
    assert a.batch == 64 and a.profile and a.trials == 3
    n2, n7, n72 = (bm.model_numbers(bm.MODELS[m]) for m in ("2b", "7b", "72b"))
    assert n2["kv_per_token"] == 28672 and n7["kv_per_token"] == 57344 and n72["kv_per_token"] == 327680
    assert abs(n2["weight_bytes"] - 3.087e9) < 2e6           # every weight once, the tied table once
    assert abs(n7["stored_bytes"] - 15.23e9) < 3e7 and abs(n7["weight_bytes"] - 14.14e9) < 3e7
    assert abs(n72["stored_bytes"] - 145.4e9) < 2e8 and abs(n72["weight_bytes"] - 142.9e9) < 2e8
    f = bm.prefill_flops(bm.MODELS["2b"], 28, 2048)
    assert abs(f["total"] - 5.73e12) < 2e10 and abs(f["attention"] - 0.36e12) < 1e10
    assert abs(bm.prefill_flops(bm.MODELS["72b"], 80, 2048)["total"] - 293e12) < 3e12
    assert bm.kernel_class("attn_decode_stream") == "attention" and bm.kernel_class("stream_ffn") == "gemm"
    assert bm.kernel_class("library_gemm") == "gemm" and bm.kernel_class("add_rmsnorm_rows") == "norm"


@pytest.mark.gpu
def test_bench_command_runs_small(tmp_path):
    """`bench decode`, `bench prefill` and `bench mixed` on two layers of the 2B sizes: JSON with the documented keys."""
    out = tmp_path / "d.json"
    p = run_cli("bench", "decode", "--model", "2b", "--layers", "2", "--batch", "4", "--ctx", "256", "--steps", "6",
                "--warmup", "3", "--trials", "2", "--profile", "--out", str(out), timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    d = json.loads(out.read_text())
    assert d["tokens_per_s"] > 0 and len(d["trials_ms"]) == 2 and d["config"]["layers"] == 2 and d["config"]["layers_of_model"] == 28
    assert d["kernels"]["gemm"]["ms"] > 0 and d["kernels"]["attention"]["frac"] > 0
    p = run_cli("bench", "mixed", "--model", "2b", "--layers", "2", "--requests", "6", "--max-running", "4", "--prompt-lo", "20",
                "--prompt-hi", "300", "--chunk", "128", "--max-new-tokens", "8", timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    m = json.loads(p.stdout.strip().splitlines()[-1])
    assert m["output_tokens"] == 48 and m["output_tokens_per_s"] > 0 and 0 < m["roofline_frac"] < 1.5
    p = run_cli("bench", "prefill", "--model", "2b", "--layers", "2", "--tokens", "512", "--trials", "2", timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert json.loads(p.stdout.strip().splitlines()[-1])["tokens"] == 512
