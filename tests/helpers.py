"""Tiny configurations, model folders and traces shared by the tests."""
from __future__ import annotations

import json
import math
import os
import random

import torch

# Two tiny Gemma 2 configurations that differ in every size and option.
TINY_A = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16,
    "intermediate_size": 128, "vocab_size": 512, "rope_theta": 10000.0, "sliding_window": 8,
    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "query_pre_attn_scalar": 16,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 64,
    "hidden_activation": "gelu_pytorch_tanh",
}
TINY_B = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 3, "hidden_size": 96, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 32,
    "intermediate_size": 320, "vocab_size": 1000, "rope_theta": 1000000.0, "sliding_window": 16,
    "attn_logit_softcapping": 20.0, "final_logit_softcapping": 15.0, "query_pre_attn_scalar": 24,
    "rms_norm_eps": 1e-5, "tie_word_embeddings": True, "max_position_embeddings": 128,
    "hidden_activation": "gelu_pytorch_tanh",
}
# Sizes that are no power of two anywhere, three query heads per kv head, an odd layer count, head size 48.
TINY_C = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 5, "hidden_size": 120, "num_attention_heads": 9, "num_key_value_heads": 3, "head_dim": 48,
    "intermediate_size": 200, "vocab_size": 777, "rope_theta": 50000.0, "sliding_window": 24,
    "attn_logit_softcapping": 30.0, "final_logit_softcapping": 0.0, "query_pre_attn_scalar": 100,
    "rms_norm_eps": 1e-4, "tie_word_embeddings": True, "max_position_embeddings": 256,
    "hidden_activation": "gelu_pytorch_tanh",
}


# Sizes the fast kernels refuse: rows that are no multiple of 16 bytes (hidden 100, inner 150) and a head size of 20,
# one kv head for five query heads, no softcaps, every layer windowed.
TINY_D = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 100, "num_attention_heads": 5, "num_key_value_heads": 1, "head_dim": 20,
    "intermediate_size": 150, "vocab_size": 333, "rope_theta": 10000.0, "sliding_window": 12,
    "attn_logit_softcapping": 0.0, "final_logit_softcapping": 0.0, "query_pre_attn_scalar": 20,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": False, "max_position_embeddings": 96,
    "hidden_activation": "gelu_pytorch_tanh", "layer_types": ["sliding_attention", "sliding_attention"],
}


# Sizes at which every fast kernel runs: head size 128 (tcgen05 prompt attention, tensor-core decode attention),
# rows of 512..1536 elements (tcgen05 products, CTA pairs for portions of more than 128 tokens), pages of 64.
TINY_E = {
    "architectures": ["Gemma2ForCausalLM"], "model_type": "gemma2",
    "num_hidden_layers": 2, "hidden_size": 512, "num_attention_heads": 6, "num_key_value_heads": 2, "head_dim": 128,
    "intermediate_size": 1536, "vocab_size": 3000, "rope_theta": 10000.0, "sliding_window": 100,
    "attn_logit_softcapping": 50.0, "final_logit_softcapping": 30.0, "query_pre_attn_scalar": 144,
    "rms_norm_eps": 1e-6, "tie_word_embeddings": True, "max_position_embeddings": 1024,
    "hidden_activation": "gelu_pytorch_tanh",
}


def write_model(folder: str, cfg_dict: dict, seed: int, dtype=torch.bfloat16, sharp: bool = False, draw: str | None = None):
    """A model folder with random weights through the framework's random-weights mode.  `draw`: 'plain' (as drawn),
    'loud' (output rows that reach the final cap) or 'sharp' (those and scores that reach the attention cap); see
    `sharpen_tensors`.  `sharp=True` is draw='sharp'."""
    draw = draw or ("sharp" if sharp else "plain")
    from kungfu_b200.api import load_config
    from kungfu_b200.weights import write_random_model
    cfg = load_config(dict(cfg_dict))
    write_random_model(folder, cfg, seed, dtype=dtype)
    with open(os.path.join(folder, "config.json"), "w") as f:      # keep the test's own dictionary
        json.dump(cfg_dict, f)
    if draw != "plain":
        sharpen(folder, cfg_dict, seed, draw)
    return folder


LOUD_FRACTION = 0.1     # of the vocabulary, at its end: ids that prompts of sharp models never hold


def quiet_vocab(cfg_dict: dict) -> int:
    """Prompts of a sharpened model draw their ids below this, so that the loud output rows are never inputs."""
    return int(cfg_dict["vocab_size"] * (1.0 - LOUD_FRACTION))


DRAWS = {"loud": dict(cap_loss=0.0, loudest=1.0), "sharp": dict(cap_loss=3.0, loudest=2.0)}


def sharpen(folder: str, cfg_dict: dict, seed: int, draw: str = "sharp") -> None:
    """`sharpen_tensors` applied to a model folder (model.safetensors is rewritten)."""
    from safetensors.torch import save_file
    tensors = {k: v.clone() for k, v in read_tensors(folder).items()}
    sharpen_tensors(cfg_dict, tensors, seed, **DRAWS[draw])
    save_file(tensors, os.path.join(folder, "model.safetensors"))


def sharpen_tensors(cfg_dict: dict, tensors: dict, seed: int, device="cpu", cap_loss: float = 3.0, loudest: float = 2.0) -> None:
    """Change random weights (a dictionary of tensors by file name, in place) so that the model's constants matter.
    With matrices of spread 0.02 every attention score is about 0.05 and every logit below 1: a softcap of 20 to 50
    is then the identity to 1e-6, and a wrong attention scale or rotation base moves the logits by less than the
    bfloat16 tolerance.  Here
    * (`cap_loss` > 0) the query and key matrices of every layer are scaled until the largest scores before the cap
      (three spreads) lose about `cap_loss` to the cap, s - cap tanh(s / cap) ~ s^3 / (3 cap^2), i.e. a factor of
      e^cap_loss in their softmax weight: for a loss of 3 a spread of 9.4 at a cap of 50, 5.1 at 20 (8 where the
      configuration has no cap);
    * (`loudest` > 0) the last tenth of the output rows (the embedding's rows when tied; those ids are kept out of the
      prompts) is scaled row by row so that the largest logit of a row before the final cap lies between 0.3 and
      `loudest` caps on the probe sequence.
    The factors are found with the plain implementation on a probe sequence, layer after layer.
    Two draws are used (`DRAWS`).  'sharp' (both, loss 3, loudest 2) for the 32-bit engine: every constant then
    moves the logits by far more than ten times the 32-bit tolerance.  It cannot serve bfloat16: scores of 20 to 40
    multiply the rounding of a hidden state (0.4 %) into several per cent of the softmax weights, so a bfloat16
    engine legitimately differs from float64 by 5 to 15 % on such a model, more than any tolerance worth having.
    'loud' (output rows only, up to one cap) keeps that difference at 1 to 1.7 % and still makes the final softcap,
    the window and the choice of sliding layers move the logits by 20 % and more; what sharp attention alone shows
    in bfloat16 (attention softcap, scale, rotation base) is covered one layer deep, where nothing multiplies the
    rounding: by the attention part's test and the attention kernels' tests
    (tests/test_oracle_sensitivity.py keeps the books)."""
    import plain_gemma2
    probe_tokens = random_tokens(min(96, cfg_dict["max_position_embeddings"]), quiet_vocab(cfg_dict), seed + 9000)
    cap = cfg_dict.get("attn_logit_softcapping") or 0.0
    spread = (3.0 * cap_loss * cap * cap) ** (1.0 / 3.0) / 3.0 if cap > 0 else 8.0 * (cap_loss / 3.0) ** (1.0 / 3.0)
    for _ in range(4 if cap_loss > 0 else 0):              # later layers see what earlier ones now produce: iterate
        pr: dict = {}
        plain_gemma2.forward(cfg_dict, tensors, probe_tokens, probe=pr, device=device)
        for l, sc in enumerate(pr["scores"]):
            f = math.sqrt(spread / max(float(sc.std()), 1e-9))
            for n in ("q_proj", "k_proj"):
                name = f"model.layers.{l}.self_attn.{n}.weight"
                tensors[name] = (tensors[name].float() * f).to(tensors[name].dtype)
    if loudest <= 0:
        return
    pr = {}
    plain_gemma2.forward(cfg_dict, tensors, probe_tokens, probe=pr, device=device)
    out_name = "lm_head.weight" if "lm_head.weight" in tensors else "model.embed_tokens.weight"
    fcap = cfg_dict.get("final_logit_softcapping") or 30.0
    V = cfg_dict["vocab_size"]
    lo = quiet_vocab(cfg_dict)
    peak = pr["logits"][:, lo:].abs().max(0).values.clamp_min(1e-9)                       # per loud row
    target = fcap * (0.3 + (loudest - 0.3) * torch.arange(V - lo, dtype=torch.float64) / max(V - lo - 1, 1))
    w = tensors[out_name]
    w[lo:] = (w[lo:].float() * (target / peak).float().to(w.device)[:, None]).to(w.dtype)


# What a test must notice: each entry changes one constant of the architecture in a copy of the configuration.
def mutations(cfg_dict: dict) -> dict:
    n = cfg_dict["num_hidden_layers"]
    out = {"attention softcap off": {"attn_logit_softcapping": 0.0},
           "final softcap off": {"final_logit_softcapping": 0.0},
           "scale from head_dim": {"query_pre_attn_scalar": cfg_dict["head_dim"]},
           "rope base x 10": {"rope_theta": cfg_dict["rope_theta"] * 10.0},
           "window + 1": {"sliding_window": cfg_dict["sliding_window"] + 1},
           "sliding on odd layers": {"layer_types": ["full_attention" if l % 2 == 0 else "sliding_attention" for l in range(n)]}}
    base_types = cfg_dict.get("layer_types") or ["sliding_attention" if l % 2 == 0 else "full_attention" for l in range(n)]
    live = {}
    for name, change in out.items():
        if all(cfg_dict.get(k, base_types if k == "layer_types" else None) == v for k, v in change.items()):
            continue                                   # the configuration already has this value: nothing to notice
        if name == "attention softcap off" and not cfg_dict.get("attn_logit_softcapping"):
            continue
        if name == "final softcap off" and not cfg_dict.get("final_logit_softcapping"):
            continue
        if name == "window + 1" and "sliding_attention" not in base_types:
            continue
        live[name] = {**cfg_dict, **change}
    return live


def read_tensors(folder: str) -> dict:
    """Tensors of a model folder through the safetensors library (not the framework's reader)."""
    from safetensors.torch import load_file
    return load_file(os.path.join(folder, "model.safetensors"))


def random_tokens(n: int, vocab: int, seed: int) -> list[int]:
    rng = random.Random(seed)
    return [rng.randrange(vocab) for _ in range(n)]


# ---- traces: lists of steps in the format bin/trace_run reads --------------------------------------------

def trace_whole(reqs: dict) -> list[dict]:
    """Each request alone and whole, all logits wanted."""
    steps = []
    for i, (rid, toks) in enumerate(reqs.items()):
        steps.append({"step": i, "entries": [{"id": rid, "tokens": list(toks), "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def trace_decode_tail(reqs: dict, tail: int = 32) -> list[dict]:
    """Most of each request in one step, the last `tail` tokens one by one."""
    steps = []
    s = 0
    for rid, toks in reqs.items():
        n = len(toks)
        head = max(1, n - tail)
        steps.append({"step": s, "entries": [{"id": rid, "tokens": list(toks[:head]), "want": list(range(head))}], "end": []})
        s += 1
        for i in range(head, n):
            steps.append({"step": s, "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": []})
            s += 1
        steps[-1]["end"] = [rid]
    return steps


def trace_chunks(reqs: dict, sizes=(7, 2, 5, 3, 2, 11, 4, 2, 9)) -> list[dict]:
    """Each request in portions of changing size, down to two tokens."""
    steps = []
    s = 0
    for rid, toks in reqs.items():
        i = 0
        c = 0
        while i < len(toks):
            n = min(sizes[c % len(sizes)], len(toks) - i)
            c += 1
            steps.append({"step": s, "entries": [{"id": rid, "tokens": list(toks[i:i + n]), "want": list(range(n))}], "end": []})
            s += 1
            i += n
        steps[-1]["end"] = [rid]
    return steps


def trace_mixed(reqs: dict, seed: int = 0, max_live: int = 4, prefill_frac: float = 0.6) -> list[dict]:
    """Up to `max_live` requests live at once: portions of some beside single tokens of others, some requests
    skipping steps; a finished request makes room for the next one."""
    rng = random.Random(seed)
    waiting = list(reqs.items())
    live: dict = {}                     # rid -> [tokens, fed]
    steps = []
    s = 0
    while waiting or live:
        while waiting and len(live) < max_live:
            rid, toks = waiting.pop(0)
            live[rid] = [list(toks), 0]
        entries, end = [], []
        for rid, (toks, fed) in list(live.items()):
            if len(live) > 1 and rng.random() < 0.2:
                continue                                    # this request sits the step out
            left = len(toks) - fed
            if fed < int(len(toks) * prefill_frac) and left > 1:
                n = min(left, rng.choice([2, 3, 5, 8, 13]))
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[fed:fed + n], "want": list(range(n))})
            live[rid][1] = fed + n
            if fed + n == len(toks):
                end.append(rid)
                del live[rid]
        if not entries:
            continue
        steps.append({"step": s, "entries": entries, "end": end})
        s += 1
    return steps


def trace_max_tokens(steps: list[dict], page: int = 64) -> int:
    """The most tokens live requests hold at any time, each request's count rounded up to `page`."""
    held: dict = {}
    best = 0
    for st in steps:
        for e in st["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        best = max(best, sum(-(-n // page) * page for n in held.values()))
        for rid in st["end"]:
            held.pop(rid, None)
    return best


def run_trace_with_runner(runner, steps: list[dict]) -> dict:
    """Drive a Runner with a trace; returns {(request, position): logits row (CPU float32)}."""
    from kungfu_b200.engine import StepEntry
    out = {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in runner.cache:
                runner.cache.add_request(e["id"])
            entries.append(StepEntry(e["id"], e["tokens"], e["want"]))
        starts = {e["id"]: runner.cache.length(e["id"]) for e in st["entries"]}
        logits = runner.step(entries)
        if logits is not None:
            logits = logits.float().cpu()
            k = 0
            for e in st["entries"]:
                for w in e["want"]:
                    out[(e["id"], starts[e["id"]] + w)] = logits[k].clone()
                    k += 1
        for rid in st["end"]:
            runner.cache.release(rid)
        runner.cache.check()
    return out
