"""The Sanarax family through the engine: checkpoints written to disk and loaded by the model directory, schedules
replayed through the scheduler, the pools and the state slots, compared with the plain oracle over whole sequences.
Covers prefill against token-by-token decoding, portions down to two tokens, unequal batches against each request
alone, pages and slots that are freed and used again, long decoding that carries every window past its kept tokens, the
residual after every layer, layers that share tensors but not caches, greedy generation through LLMEngine.generate, and
the trace replay program."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import sanarax_ref as R
import sanarax_util as U

pytestmark = pytest.mark.gpu

CONFIGS = {"a": U.cfg_a, "b": U.cfg_b, "c": U.cfg_c, "d": U.cfg_d, "e": U.cfg_e, "f": U.cfg_f}


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, make in CONFIGS.items():
        cfg = make()
        W = R.random_model(cfg, seed=len(name) + ord(name))
        out[name] = (cfg, W, U.save_checkpoint(tmp_path_factory.mktemp("sanarax_" + name), cfg, W))
    return out


_oracle_cache = {}


def _oracle(cfg, W, toks):
    key = (id(W), tuple(toks))
    if key not in _oracle_cache:
        _oracle_cache[key] = U.oracle_logits(cfg, W, toks)
    return _oracle_cache[key]


def _check(got, cfg, W, reqs, dtype, what=""):
    for rid, toks in reqs.items():
        err = U.rel_err(got[rid], _oracle(cfg, W, toks), dtype)
        assert err <= U.TOL[dtype], f"{what} request {rid}: error {err:.3e} above {U.TOL[dtype]:.1e} ({dtype})"


@pytest.mark.parametrize("name", sorted(CONFIGS))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_prompt_and_token_by_token(cuda, models, name, dtype):
    cfg, W, path = models[name]
    eng = U.make_engine(path, dtype)
    reqs = {"p": U.tokens(70, cfg["vocab"], 1), "q": U.tokens(1, cfg["vocab"], 2)}
    whole = U.replay(eng, reqs, [[("p", 70)], [("q", 1)]])
    _check(whole, cfg, W, reqs, dtype, "whole")
    single = U.replay(eng, {"p": reqs["p"]}, [[("p", 1)] for _ in range(70)])          # every token a step of its own
    _check(single, cfg, W, {"p": reqs["p"]}, dtype, "token by token")
    assert U.rel_err(single["p"], whole["p"], dtype) <= U.TOL[dtype]
    eng.close()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_residual_after_every_layer(cuda, models, name):
    cfg, W, path = models[name]
    eng = U.make_engine(path, "float32", eager=True)
    toks = U.tokens(29, cfg["vocab"], 3)
    eng.model.capture = []
    eng.replay_step([("r", toks, [])], ["r"])
    trail = []
    R.forward(cfg, W, toks, trail)
    assert len(eng.model.capture) == len(cfg["layers"])
    for i, x in enumerate(eng.model.capture):
        err = float((x.double().cpu() - trail[i]).abs().max() / trail[i].abs().max())
        assert err <= 1e-4, f"layer {i}: {err:.3e}"
    eng.close()


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_of_many_sizes(cuda, models, name):
    """Cuts inside pages (16), inside and at the edges of the windows (1, 5, 8, 9, 16, 17, 40, 50) and of the kept prefixes,
    portions of 2 and 3."""
    cfg, W, path = models[name]
    eng = U.make_engine(path, "float32")
    toks = U.tokens(131, cfg["vocab"], 7)
    for cuts in ([2, 3, 11, 17, 31, 2, 33, 30, 2], [64, 2, 2, 63], [15, 1, 1, 16, 32, 1, 65], [6, 1, 13, 43, 1, 67]):
        assert sum(cuts) == 131
        got = U.replay(eng, {"r": toks}, [[("r", n)] for n in cuts])
        _check(got, cfg, W, {"r": toks}, "float32", f"cuts {cuts}")
    eng.close()


@pytest.mark.parametrize("name,dtype", [("a", "float32"), ("b", "float32"), ("c", "float32"), ("d", "float32"), ("e", "float32"),
                                        ("f", "float32"), ("a", "bfloat16"), ("c", "bfloat16"), ("e", "bfloat16"), ("f", "bfloat16")])
def test_unequal_batches_with_reuse_of_pages_and_slots(cuda, models, name, dtype):
    """Up to four live requests, prompt portions beside single tokens; requests leave and new ones take over their pages
    and state slots (a pool of 15 pages for ~320 tokens in total).  Every request equals the oracle over its own tokens,
    and equals itself run alone."""
    cfg, W, path = models[name]
    V = cfg["vocab"]
    reqs = {"a": U.tokens(90, V, 1), "b": U.tokens(33, V, 2), "c": U.tokens(1, V, 3), "d": U.tokens(47, V, 4),
            "e": U.tokens(60, V, 5), "f": U.tokens(52, V, 6), "g": U.tokens(40, V, 7)}
    sched = [[("a", 30), ("b", 31), ("c", 1)],                       # c lives for one step
             [("a", 1), ("b", 1), ("d", 17)],
             [("a", 1), ("b", 1), ("d", 2), ("e", 3)],               # b ends: its slot and pages go back
             [("a", 28), ("d", 1), ("e", 1), ("f", 20)],             # f takes b's slot
             [("a", 1), ("d", 27), ("e", 40), ("f", 1)],             # d ends
             [("a", 29), ("e", 16), ("f", 31), ("g", 2)],            # a, e, f end; g took d's slot
             [("g", 1)], [("g", 1)], [("g", 36)]]
    eng = U.make_engine(path, dtype, max_tokens=15 * 16)
    got = U.replay(eng, reqs, sched)
    assert eng.sched.num_free_blocks == eng.num_blocks and eng.sched.num_running == 0
    _check(got, cfg, W, reqs, dtype, "mixed")
    for rid, toks in reqs.items():
        alone = U.replay(eng, {rid: toks}, [[(rid, len(toks))]])
        assert U.rel_err(got[rid], alone[rid], dtype) <= (1e-5 if dtype == "float32" else 2e-2), f"request {rid} against itself alone"
    eng.close()


@pytest.mark.parametrize("name,eager", [("a", False), ("a", True), ("c", False), ("f", False)])
def test_long_decoding_through_graph_and_eager_steps(cuda, models, name, eager):
    """A 20-token prompt then 230 single-token steps (the decode-only step is a CUDA graph unless eager), beside a second
    request that joins late: every window slides far past its kept tokens while decoding and every state is carried 250
    steps."""
    cfg, W, path = models[name]
    reqs = {"x": U.tokens(250, cfg["vocab"], 21), "y": U.tokens(120, cfg["vocab"], 22)}
    sched = [[("x", 20)]] + [[("x", 1)] for _ in range(110)] + [[("x", 1), ("y", 1)] for _ in range(120)]
    eng = U.make_engine(path, "float32", eager=eager)
    got = U.replay(eng, reqs, sched)
    _check(got, cfg, W, reqs, "float32", "long decode")
    assert eng.stats.decode_steps >= 229 and (eager or len(eng._graphs) >= 2)
    eng.close()


@pytest.mark.parametrize("name", ["e", "f"])
def test_long_portions_rebuild_keys_and_values_per_head(cuda, models, name):
    """bf16 steps with 256 prompt rows and more leave the latent space in the latent layers: alone, beside decode rows and
    another portion, and with 300 tokens of context before the portion.  The logits equal the oracle's and those of the
    same requests cut into small portions (which stay in the latent space)."""
    cfg, W, path = models[name]
    V = cfg["vocab"]
    reqs = {"a": U.tokens(600, V, 41), "b": U.tokens(330, V, 42), "c": U.tokens(50, V, 43)}
    long_sched = [[("a", 300), ("c", 20)], [("a", 1), ("b", 290), ("c", 1)], [("a", 280), ("b", 1), ("c", 29)], [("a", 19), ("b", 39)]]
    eng = U.make_engine(path, "bfloat16", max_tokens=1024)
    seen = []
    plan = eng.model._prompt_plan
    eng.model._prompt_plan = lambda pf: seen.append(plan(pf)) or seen[-1]
    got = U.replay(eng, reqs, long_sched)
    assert [p is not None for p in seen] == [True, True, True, False]
    _check(got, cfg, W, reqs, "bfloat16", "long portions")
    small = U.replay(eng, reqs, [[("a", 100)]] * 6 + [[("b", 110)]] * 3 + [[("c", 50)]])
    assert all(p is None for p in seen[4:])
    for rid in reqs:
        assert U.rel_err(got[rid], small[rid], "bfloat16") <= 2e-2, f"request {rid}: long against short portions"
    eng.close()


def test_layers_that_share_tensors_keep_caches_of_their_own(cuda, models):
    """The model with weights_of equals the model in which those layers carry copies of the tensors under their own names,
    through portions and single tokens."""
    cfg, W, path = models["a"]
    flat, W2 = json.loads(json.dumps(cfg)), dict(W)
    for i, L in enumerate(flat["layers"]):
        j = L.pop("weights_of", None)
        if j is not None:
            for k, t in W.items():
                if k.startswith(f"l{j}."):
                    W2[f"l{i}." + k.split(".", 1)[1]] = t.clone()
    path2 = U.save_checkpoint(path.parent / "flat", flat, W2)
    toks = U.tokens(60, cfg["vocab"], 4)
    sched = [[("r", 25)], [("r", 2)]] + [[("r", 1)]] * 8 + [[("r", 25)]]
    outs = []
    for p in (path, path2):
        eng = U.make_engine(p, "float32")
        assert len(eng.model.k_cache) == 2 and len(eng.model.state) == 2
        outs.append(U.replay(eng, {"r": toks}, sched)["r"])
        eng.close()
    assert U.rel_err(outs[0], outs[1]) <= 1e-6
    sizes = []
    for p in (path, path2):
        eng = U.make_engine(p, "float32")
        sizes.append(eng.model.weight_bytes())
        eng.close()
    assert sizes[0] < sizes[1]


def test_block_size_and_pool_do_not_change_the_logits(cuda, models):
    cfg, W, path = models["c"]
    toks = U.tokens(77, cfg["vocab"], 9)
    ref = None
    for bs in (8, 16, 32):
        eng = U.make_engine(path, "float32", max_tokens=96, block_size=bs)
        got = U.replay(eng, {"r": toks}, [[("r", 50)], [("r", 2)], [("r", 25)]])["r"]
        _check({"r": got}, cfg, W, {"r": toks}, "float32", f"block size {bs}")
        ref = got if ref is None else ref
        assert U.rel_err(got, ref) <= 1e-5
        eng.close()


@pytest.mark.parametrize("name", ["a", "d"])
def test_greedy_generation_through_the_engine(cuda, models, name):
    """LLMEngine.generate (scheduler policy, chunked prefill, CUDA-graph decode, b2_sample at temperature 0) continues
    three prompts exactly as the oracle's argmax does, with fewer sequence slots than requests."""
    from b200attn.engine import SamplingParams
    cfg, W, path = models[name]
    eng = U.make_engine(path, "float32", max_num_seqs=2)
    prompts = [U.tokens(n, cfg["vocab"], 30 + n) for n in (5, 19, 1)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
    for p, out in zip(prompts, outs):
        seq = list(p)
        for k in range(12):
            lg = U.oracle_logits(cfg, W, seq)[-1]
            top2 = torch.topk(lg, 2).values
            if float(top2[0] - top2[1]) < 1e-2 * float(lg.abs().max()):
                break                                               # a near tie for a sampler that reads the logits in 16 bits
            assert out[k] == int(lg.argmax()), f"token {k} of prompt of {len(p)}"
            seq.append(out[k])
    eng.close()


def test_random_init_and_checkpoint_shape_check(cuda, tmp_path, models):
    """Without weights in the directory the engine serves seeded random weights of the configuration; a checkpoint
    whose shapes contradict config.json, or that lacks a tensor, is refused."""
    cfg, W, _ = models["b"]
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    eng = U.make_engine(tmp_path, "bfloat16")
    lg = eng.replay_step([("r", U.tokens(9, cfg["vocab"], 1), [8])], ["r"])
    assert lg.shape == (1, cfg["vocab"]) and bool(torch.isfinite(lg).all())
    eng.close()
    bad = dict(W)
    bad["l0.mix.sink"] = torch.zeros(5, dtype=torch.bfloat16)
    U.save_checkpoint(tmp_path / "bad", cfg, bad)
    with pytest.raises(ValueError, match="sink"):
        U.make_engine(tmp_path / "bad", "bfloat16")
    less = {k: v for k, v in W.items() if k != "l1.mix.dq.norm"}
    U.save_checkpoint(tmp_path / "less", cfg, less)
    with pytest.raises(ValueError, match="lacks"):
        U.make_engine(tmp_path / "less", "bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_program(cuda, models, tmp_path, dtype):
    """bin/trace_run as a subprocess: steps on standard input, one `done` line per step, logits files for the wanted rows."""
    cfg, W, path = models["d"]
    root = Path(__file__).resolve().parent.parent
    a, b = U.tokens(40, cfg["vocab"], 11), U.tokens(9, cfg["vocab"], 12)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:33], "want": [0, 32]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[33:34], "want": [0]}, {"id": "b", "tokens": b, "want": [8]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": a[34:], "want": []}], "end": ["a"]}]
    out = tmp_path / "out"
    out.mkdir()
    env = {k: v for k, v in os.environ.items() if k != "B200ATTN_LIB"}
    r = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(path), "--dtype", dtype, "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                       text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not (out / "2.f32").exists()
    la, lb = U.oracle_logits(cfg, W, a), U.oracle_logits(cfg, W, b)
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1))
    tol = U.TOL[dtype] * (1 if dtype == "float32" else 3)
    assert U.rel_err(got0, la[[0, 32]]) <= tol and U.rel_err(got1, torch.stack([la[33], lb[8]])) <= tol


def test_server_serves_a_model_directory(cuda, models):
    """`python -m b200attn.server --model DIR --dtype float32`: the family comes from config.json, completions are the
    oracle's greedy continuation of a token-id prompt."""
    import socket
    import time

    import requests
    cfg, W, path = models["b"]
    sock = socket.socket()
    sock.bind(("127.0.0.1", 0))
    port = sock.getsockname()[1]
    sock.close()
    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root / "vllm-backend-public_b200"))
    proc = subprocess.Popen([sys.executable, "-m", "b200attn.server", "--model", str(path), "--dtype", "float32", "--port", str(port),
                             "--host", "127.0.0.1", "--max-num-seqs", "4", "--max-model-len", "256",
                             "--num-gpu-blocks-override", "80", "--served-model-name", "sanarax-test"], env=env,
                            stdout=subprocess.PIPE, stderr=subprocess.STDOUT)
    base = f"http://127.0.0.1:{port}"
    try:
        for _ in range(600):
            if proc.poll() is not None:
                raise RuntimeError("server exited: " + proc.stdout.read().decode()[-2000:])
            try:
                if requests.get(base + "/health", timeout=1).status_code == 200:
                    break
            except requests.RequestException:
                pass
            time.sleep(0.2)
        else:
            raise RuntimeError("server did not become healthy")
        body = None
        for seed in range(80, 90):                                  # a prompt whose six greedy steps all have a clear winner
            prompt = U.tokens(11, cfg["vocab"], seed)
            seq, clear = list(prompt), True
            for _ in range(6):
                lg = U.oracle_logits(cfg, W, seq)[-1]
                top2 = torch.topk(lg, 2).values
                clear = clear and float(top2[0] - top2[1]) > 1e-2 * float(lg.abs().max())
                seq.append(int(lg.argmax()))
            if not clear:
                continue
            r = requests.post(base + "/v1/completions", json={"model": "sanarax-test", "prompt": prompt, "max_tokens": 6,
                                                              "temperature": 0.0, "ignore_eos": True}, timeout=60)
            assert r.status_code == 200, r.text
            body = r.json()
            assert body["usage"]["prompt_tokens"] == 11 and body["usage"]["completion_tokens"] == 6
            want = bytes(t % 256 for t in seq[11:]).decode("utf-8", errors="replace")      # the byte tokenizer's text
            assert body["choices"][0]["text"] == want
            break
        assert body is not None
    finally:
        proc.terminate()
        try:
            proc.wait(20)
        except subprocess.TimeoutExpired:
            proc.kill()
