"""The command line: ``random-model`` writes a folder the loader accepts; ``generate`` (GPU) gives the tokens of
the plain implementation."""
import json
import os
import subprocess
import sys

import pytest
import torch

import helpers as H
import plain_model as P

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DINFER = os.path.join(ROOT, "bin", "dinfer")


def run(*args):
    return subprocess.run([sys.executable, DINFER, *args], capture_output=True, text=True, timeout=600)


def test_random_model_writes_a_loadable_folder(tmp_path):
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(H.TINY_A))
    out = tmp_path / "model"
    r = run("random-model", "--config", str(cfg_path), "--out", str(out), "--seed", "3", "--std", "0.05",
            "--norm-jitter", "0.1", "--dtype", "float32")
    assert r.returncode == 0, r.stderr
    assert sorted(os.listdir(out)) == ["config.json", "model.safetensors"]
    from dinfer_b200.config.model_config import Qwen3Config, read_config_json
    from dinfer_b200.weights.loader import SafetensorsSource
    cfg = Qwen3Config.from_dict(read_config_json(str(out)))
    assert cfg.hidden_size == H.TINY_A["hidden_size"]
    src = SafetensorsSource(str(out))
    try:
        names = set(src.names())
    finally:
        src.close()
    assert "model.embed_tokens.weight" in names and "model.layers.1.mlp.down_proj.weight" in names
    assert "lm_head.weight" not in names                       # tied embeddings: no separate head
    # the same seed gives the same file
    out2 = tmp_path / "model2"
    assert run("random-model", "--config", str(cfg_path), "--out", str(out2), "--seed", "3", "--std", "0.05",
               "--norm-jitter", "0.1", "--dtype", "float32").returncode == 0
    assert (out / "model.safetensors").read_bytes() == (out2 / "model.safetensors").read_bytes()


def test_usage_errors():
    assert run("generate").returncode != 0                      # --model or --random-weights is required
    assert run("generate", "--model", "x", "--random-weights", "y").returncode != 0     # not both
    assert run("no-such-command").returncode != 0
    r = run("generate", "--help")
    assert r.returncode == 0 and "--max-num-batched-tokens" in r.stdout and "--enable-prefix-caching" in r.stdout
    assert run("generate", "--model", "x", "--split-norms", "sometimes").returncode != 0     # on, off or auto


@pytest.mark.gpu
def test_generate_gives_the_plain_tokens(tmp_path):
    d = H.make_model_dir(str(tmp_path / "b"), H.TINY_B, *H.INIT["B"], torch.float32)
    W = H.load_plain_weights(d)
    prompts = [[5, 17, 3, 9], [100, 2, 77, 300, 11, 8, 9, 40, 41]]
    r = run("generate", "--model", d, "--dtype", "float32", "--max-model-len", "64", "--max-num-seqs", "2",
            "--num-blocks", "16", "--prompt-ids", ",".join(map(str, prompts[0])), "--prompt-ids",
            " ".join(map(str, prompts[1])), "--max-tokens", "7", "--temperature", "0", "--ignore-eos")
    assert r.returncode == 0, r.stderr
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 2
    for line, p in zip(lines, prompts):
        assert line["output_ids"] == P.greedy_generate(W, H.TINY_B, p, 7)
        assert line["finish_reason"] == "length"


@pytest.mark.gpu
def test_generate_with_random_weights_needs_no_files(tmp_path):
    """``--random-weights config.json``: the weights are drawn on the device from the seed; the same seed gives the
    same tokens, another seed other tokens."""
    cfg_path = tmp_path / "cfg.json"
    cfg_path.write_text(json.dumps(H.TINY_B))

    def tokens(seed):
        r = run("generate", "--random-weights", str(cfg_path), "--weights-seed", str(seed), "--weights-std", "0.03",
                "--weights-norm-jitter", "0.2", "--dtype", "float32", "--max-model-len", "64", "--max-num-seqs", "2",
                "--num-blocks", "16", "--prompt-ids", "5,17,3,9", "--max-tokens", "8", "--temperature", "0", "--ignore-eos")
        assert r.returncode == 0, r.stderr
        return [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")][0]["output_ids"]

    a, b, c = tokens(1), tokens(1), tokens(2)
    assert len(a) == 8 and a == b and a != c


@pytest.mark.gpu
def test_generate_with_the_norms_taken_apart_where_measured_faster(tmp_path):
    """``--split-norms auto`` (and plain ``--split-norms`` = on) in bfloat16: the run goes through and gives as many
    tokens as asked, ids within the vocabulary."""
    d = H.make_model_dir(str(tmp_path / "d"), H.TINY_D, *H.INIT["D"], torch.bfloat16)
    for flag in (["--split-norms", "auto"], ["--split-norms"]):
        r = run("generate", "--model", d, "--dtype", "bfloat16", "--max-model-len", "64", "--max-num-seqs", "2",
                "--num-blocks", "16", "--prompt-ids", "5,17,3,9", "--max-tokens", "6", "--temperature", "0",
                "--ignore-eos", *flag)
        assert r.returncode == 0, r.stderr
        line = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")][0]
        assert len(line["output_ids"]) == 6 and all(0 <= t < H.TINY_D["vocab_size"] for t in line["output_ids"])
