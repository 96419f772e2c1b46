"""The command line: inspect and describe run anywhere; generate, score and bench need the GPU."""
import json
import os
import subprocess
import sys

import pytest
import torch

import helpers
import plain_gemma2

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KUNGFU = [sys.executable, os.path.join(ROOT, "bin", "kungfu")]


def run(args, **kw):
    return subprocess.run(KUNGFU + args, capture_output=True, text=True, timeout=600, **kw)


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    return helpers.write_model(str(tmp_path_factory.mktemp("cli") / "m"), helpers.TINY_B, seed=17, dtype=torch.bfloat16)


def test_random_weights_and_inspect(tmp_path, model_dir):
    cfg_path = tmp_path / "config.json"
    cfg_path.write_text(json.dumps(helpers.TINY_A))
    out = tmp_path / "model"
    p = run(["random-weights", "--config", str(cfg_path), "--out", str(out), "--seed", "3"])
    assert p.returncode == 0 and os.path.exists(out / "model.safetensors") and os.path.exists(out / "config.json")
    p = run(["inspect", str(out), "--json"])
    assert p.returncode == 0, p.stderr
    doc = json.loads(p.stdout)
    assert doc["architecture"] == "Gemma2ForCausalLM" and doc["tensors"] == 24 and doc["layers"] == 2
    assert [s["window"] for s in doc["states"]] == [8, None] and doc["states"][0]["kind"] == "kv_cache"
    assert doc["missing"] == [] and doc["unexpected"] == []
    # a tensor nobody claims makes inspect fail, as the reference's does (crates/kungfu/src/main.rs:262-265)
    from kungfu_b200.weights import write_safetensors
    tensors = dict(helpers.read_tensors(str(out)))
    tensors["stray.weight"] = torch.zeros(3)
    write_safetensors(str(out / "model.safetensors"), tensors)
    p = run(["inspect", str(out)])
    assert p.returncode == 1 and "stray.weight" in p.stderr


def test_describe():
    p = run(["describe"])
    assert p.returncode == 0, p.stderr
    doc = json.loads(p.stdout)
    assert "Gemma2ForCausalLM" in doc["architectures"] and "paged_attention" in doc["parts"]["mixer"]
    assert {"--model", "--ctx", "--batch", "--temperature"} <= {x["flag"] for x in doc["params"]}


def test_generate_needs_ids_and_refuses_cpu(model_dir):
    assert run(["generate", "--model", model_dir]).returncode != 0
    p = run(["generate", "--model", model_dir, "--ids", "[1, 2]", "--backend", "cpu"])
    assert p.returncode != 0 and "cpu" in p.stderr


@pytest.mark.gpu
def test_generate_score_bench(model_dir):
    cfg = helpers.TINY_B
    tensors = helpers.read_tensors(model_dir)
    ids = helpers.random_tokens(19, cfg["vocab_size"], 4)
    p = run(["generate", "--model", model_dir, "--ids", json.dumps(ids), "--max-tokens", "6", "--dtype", "float32", "--emit-ids",
             "--ctx", "128", "--ignore-eos"])
    assert p.returncode == 0, p.stderr[-2000:]
    doc = json.loads(p.stdout.strip().split("\n")[-1])
    assert doc["prompt"] == ids and doc["generated"] == plain_gemma2.greedy(cfg, tensors, ids, 6)
    # score: greedy prediction at every position, first 7 ids as one batch and the rest one by one
    p = run(["score", "--model", model_dir, "--ids", json.dumps(ids), "--prefix", "7", "--dtype", "float32", "--ctx", "128"])
    assert p.returncode == 0, p.stderr[-2000:]
    pred = json.loads(p.stdout.strip().split("\n")[-1])["predictions"]
    want = torch.argmax(plain_gemma2.forward(cfg, tensors, ids), dim=-1).tolist()
    assert pred == want
    p = run(["score", "--model", model_dir, "--ids", json.dumps(ids), "--topk", "3", "--dtype", "float32", "--ctx", "128"])
    top3 = json.loads(p.stdout.strip().split("\n")[-1])["predictions"]
    assert [t[0] for t in top3] == want and all(len(t) == 3 for t in top3)
    p = run(["bench", "--model", model_dir, "--pp", "32", "--tg", "8", "--reps", "2", "--ctx", "128", "--batch", "16", "--trace"])
    assert p.returncode == 0, p.stderr[-2000:]
    assert "pp32" in p.stdout and "tg8" in p.stdout
    assert "kernel times, decode step" in p.stderr and "paged_attention" in p.stderr
    # temperature sampling with events
    p = run(["generate", "--model", model_dir, "--ids", json.dumps(ids), "--max-tokens", "5", "--temperature", "0.8", "--seed", "3",
             "--ctx", "128", "--events"])
    assert p.returncode == 0 and "kungfu event=ready" in p.stderr and "kungfu event=request" in p.stderr
    assert "kungfu event=plan " in p.stderr and "kungfu event=alloc pool=cuda0 kind=weights" in p.stderr
    assert "kind=cache" in p.stderr
    # no model folder: the weights a folder written with the same seed would hold, drawn on the device
    cfg_path = os.path.join(model_dir, "config.json")
    p = run(["generate", "--config", cfg_path, "--random-weights", "--weights-seed", "17", "--ids", json.dumps(ids), "--max-tokens", "6",
             "--dtype", "float32", "--ctx", "128", "--ignore-eos"])
    assert p.returncode == 0, p.stderr[-2000:]
    assert json.loads(p.stdout.strip().split("\n")[-1])["generated"] == plain_gemma2.greedy(cfg, tensors, ids, 6)
