"""The command line: option names and defaults of the reference, inspect without a GPU."""
import json
import os
import subprocess
import sys

import pytest

import helpers
from llama_rs_metal_b200 import cli

CLI = os.path.join(helpers.ROOT, "bin", "llama-cli")


def test_sampling_options_have_the_reference_defaults():
    # crates/llama-cli/src/main.rs:79-93
    args = cli.build_parser().parse_args(["generate", "-m", "x", "-p", "1,2"])
    assert (args.max_tokens, args.temperature, args.top_k, args.top_p, args.repeat_penalty, args.seed) == \
           (256, 0.8, 40, 0.95, 1.0, 42)
    assert args.context == 0 and args.memory_mib is None and args.float_weights_f32 is False
    args = cli.build_parser().parse_args(["generate", "--model", "x", "--prompt", "@f", "-n", "5", "-c", "64",
                                          "--float-weights-f32", "--memory-mib", "100"])
    assert (args.max_tokens, args.context, args.float_weights_f32, args.memory_mib) == (5, 64, True, 100)


def test_prompts_are_token_ids(tmp_path):
    assert cli._parse_prompt("1, 2,3") == [1, 2, 3]
    (tmp_path / "ids.txt").write_text("7 8\n9\n")
    assert cli._parse_prompt("@" + str(tmp_path / "ids.txt")) == [7, 8, 9]


def test_inspect_and_random_run_without_a_gpu(tmp_path):
    config = tmp_path / "config.json"
    config.write_text(json.dumps(helpers.TINY["B"]["config"]))
    out = subprocess.run([sys.executable, CLI, "random", "--config", str(config), "--out", str(tmp_path / "m"),
                          "--seed", "7", "--std", "0.05"], capture_output=True, text=True,
                         env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert out.returncode == 0, out.stderr
    out = subprocess.run([sys.executable, CLI, "inspect", str(tmp_path / "m"), "--tensors"],
                         capture_output=True, text=True, env={**os.environ, "CUDA_VISIBLE_DEVICES": ""})
    assert out.returncode == 0, out.stderr
    report = json.loads(out.stdout)
    assert report["format"] == "safetensors" and report["config"]["num_hidden_layers"] == 3
    assert report["tensor_count"] == 3 * 9 + 3
    entry = report["tensors"]["model.layers.2.mlp.down_proj.weight"]
    assert entry == {"dimensions": [96, 256], "storage_bytes": 96 * 256 * 2, "encoding": "bfloat16"}
    assert report["weight_bytes"] == sum(t["storage_bytes"] for t in report["tensors"].values())
    bad = subprocess.run([sys.executable, CLI, "inspect", str(tmp_path / "nothing")], capture_output=True, text=True)
    assert bad.returncode == 1 and bad.stderr.startswith("error:")


@pytest.mark.gpu
def test_generate_prints_token_ids_and_finish_reasons(model_dirs):
    out = subprocess.run([sys.executable, CLI, "generate", "-m", model_dirs["A"], "-p", "1,2,3", "-p", "9",
                          "-n", "4", "--temperature", "0", "-c", "64", "--float-weights-f32"],
                         capture_output=True, text=True)
    assert out.returncode == 0, out.stderr
    lines = out.stdout.strip().splitlines()
    tokens = [l.split("\t") for l in lines if "\t" in l]
    finished = [json.loads(l) for l in lines if l.startswith("{")]
    assert len(tokens) == 8 and len(finished) == 2
    assert all(f["reason"] == "length" and f["tokens"] == 4 for f in finished)
    assert finished[0]["ids"] == [int(t) for r, t in tokens if r == "0"]
    assert "context 64" in out.stderr
