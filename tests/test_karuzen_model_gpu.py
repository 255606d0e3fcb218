"""Karuzen through the runner and the engine: logits of every position against the plain fp32 oracle, whatever the
schedule - whole prompts, token-by-token decoding, portions down to two tokens, mixed batches, reused pages - plus greedy
generation through LLMEngine's own scheduler.  Small configurations with sizes that differ from one another (dim, vdim,
latent ranks, per-layer head counts), a layer without feed-forward, top = 1, a router without a shared expert, a looped
block that does not start at layer 0."""
import importlib

import numpy as np
import pytest
import torch

from oracle import karuzen_oracle as K

pytestmark = pytest.mark.gpu
BLOCK = 16


def cfg_a(all_experts=False):
    """all_experts: every expert is chosen (top = experts), so that no bf16 rounding of a router's input can flip a near-tie
    between two experts - a flip changes a position by far more than rounding, and every later position attends to it.
    The bf16 rigs use it; the choice itself is checked in fp32 here and in both formats at the kernel level."""
    ea, eb = ((3, 3), (2, 2)) if all_experts else ((6, 2), (5, 1))
    return K.make_config(vocab=320, width=192, layers=[
        {"type": "latent_attention", "mixer": K.mixer_cfg(4, 32, 48, 96, 40, 0.2), "mlp": K.dense_cfg(160)},
        {"type": "latent_attention", "mixer": K.mixer_cfg(3, 48, 32, 40, 72, 0.15), "mlp": K.moe_cfg(ea[0], ea[1], 48, 1.5, 80)},
        {"type": "latent_attention", "mixer": K.mixer_cfg(2, 64, 64, 64, 64, 0.125), "mlp": None},
        {"type": "latent_attention", "mixer": K.mixer_cfg(5, 24, 40, 136, 24, 0.3), "mlp": K.moe_cfg(eb[0], eb[1], 72, 0.7, 0)},
    ], loop={"start": 1, "stop": 3, "times": 2})


def cfg_b():
    """No loop, one expert, vocab and width that are multiples of nothing."""
    return K.make_config(vocab=203, width=100, layers=[
        {"type": "latent_attention", "mixer": K.mixer_cfg(1, 16, 8, 24, 8, 0.25), "mlp": K.moe_cfg(1, 1, 40, 2.0, 24)},
        {"type": "latent_attention", "mixer": K.mixer_cfg(7, 8, 16, 200, 104, 0.35), "mlp": K.dense_cfg(72)},
    ], loop=None)


class Rig:
    def __init__(self, cfg, dtype, blocks=40, seed=0, chunked=True):
        self.eng = importlib.import_module("nano-vllm-candle_b200.engine")
        self.cfg, self.dtype = cfg, dtype
        self.w = K.make_weights(cfg, seed)
        self.oracle = K.KaruzenOracle(cfg, self.w)
        self.ctx = self.eng.DeviceContext(0)
        T = blocks * BLOCK
        self.runner = self.eng.ModelRunner.from_config(self.ctx, cfg, self.w.items(), num_kvcache_blocks=blocks, kvcache_block_size=BLOCK,
                                                       max_num_seqs=4, max_num_batched_tokens=T, max_model_len=T, dtype=dtype,
                                                       max_logit_rows=T)
        sc = self.eng.SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=T, eos=-1, num_kvcache_blocks=blocks,
                                      kvcache_block_size=BLOCK, enable_chunked_prefill=chunked, max_model_len=T)
        self.engine = self.eng.LLMEngine(self.eng.Scheduler(sc), self.runner, greedy=True)
        # error of a position: rms over the vocabulary of the mean-free logit difference, relative to the logits' own rms
        self.tol = 1e-4 if dtype == "float32" else 0.03

    def close(self):
        self.engine.close()
        self.runner.close()
        self.ctx.close()

    def want(self, tokens):
        return self.oracle.forward(tokens).numpy()

    def replay(self, prompts, schedule):
        """schedule: steps of [(request, count)]; every position's logits are collected; requests end when exhausted."""
        live, at = {}, {k: 0 for k in prompts}
        got = {k: np.zeros((len(v), self.cfg["vocab"]), np.float32) for k, v in prompts.items()}
        for step in schedule:
            entries = []
            for name, n in step:
                if name not in live:
                    live[name] = self.engine.open_request()
                entries.append((live[name], prompts[name][at[name]:at[name] + n], list(range(n))))
            lg = self.engine.step_forced(entries)
            row = 0
            for name, n in step:
                got[name][at[name]:at[name] + n] = lg[row:row + n]
                row += n
                at[name] += n
                if at[name] == len(prompts[name]):
                    self.engine.close_request(live.pop(name))
        assert all(at[k] == len(v) for k, v in prompts.items())
        return got

    def check(self, prompts, schedule):
        got = self.replay(prompts, schedule)
        for k, toks in prompts.items():
            err = self.rel_err(got[k], self.want(toks))
            bad = err >= self.tol
            assert not bad.any(), \
                f"{k}: {int(bad.sum())} of {len(toks)} positions over {self.tol}, first {int(np.argmax(bad))}, worst {err.max():.4g}"

    @staticmethod
    def rel_err(got, want):
        d = got - want
        d = d - d.mean(-1, keepdims=True)
        w = want - want.mean(-1, keepdims=True)
        return np.sqrt((d * d).mean(-1)) / np.sqrt((w * w).mean(-1))


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def rig(request):
    r = Rig(cfg_a(all_experts=request.param == "bfloat16"), request.param)
    yield r
    r.close()


def test_whole_prompts_and_first_tokens(rig):
    V = rig.cfg["vocab"]
    rig.check({"one": toks(1, V, 1)}, [[("one", 1)]])
    rig.check({"p": toks(83, V, 2)}, [[("p", 83)]])
    rig.check({"page": toks(2 * BLOCK, V, 3)}, [[("page", 2 * BLOCK)]])


def test_residual_stream_after_every_layer_run(rig):
    p = toks(21, rig.cfg["vocab"], 4)
    tap = rig.runner.tap_residual(len(p))
    sid = rig.engine.open_request()
    rig.engine.step_forced([(sid, p, [0])])
    rig.engine.close_request(sid)
    res = []
    rig.oracle.forward(p, residuals=res)
    assert tap.shape[0] == len(res) == 6       # layer 0, (1, 2) twice, 3
    for k, want in enumerate(res):
        assert np.abs(tap[k] - want.numpy()).max() < (2e-4 if rig.dtype == "float32" else 0.3), f"layer run {k}"


def test_prefill_then_token_by_token(rig):
    p = toks(70, rig.cfg["vocab"], 5)
    rig.check({"d": p}, [[("d", 30)]] + [[("d", 1)]] * 40)
    rig.check({"d": p}, [[("d", 1)]] * 70)             # decoding from the very first token, across page borders


def test_portions_of_many_sizes(rig):
    p = toks(121, rig.cfg["vocab"], 6)
    sizes = [2, 14, 16, 1, 17, 2, 31, 3, 33, 2]        # cuts before, at and after page borders
    assert sum(sizes) == 121
    rig.check({"c": p}, [[("c", n)] for n in sizes])


def test_long_decoding(rig):
    p = toks(260, rig.cfg["vocab"], 7)
    rig.check({"l": p}, [[("l", 5)]] + [[("l", 1)]] * 255)


def test_mixed_batches_equal_each_request_alone(rig):
    V = rig.cfg["vocab"]
    pr = {"a": toks(90, V, 8), "b": toks(37, V, 9), "c": toks(3, V, 10), "d": toks(64, V, 11)}
    sched = [[("a", 40), ("b", 2)], [("a", 1), ("b", 20), ("c", 1)], [("a", 1), ("c", 1), ("d", 64)], [("a", 17), ("b", 1), ("c", 1)],
             [("a", 1), ("b", 14)]] + [[("a", 1)]] * 30
    assert all(sum(n for s in sched for k, n in s if k == name) == len(p) for name, p in pr.items())
    rig.check(pr, sched)


def test_pages_are_freed_and_used_again(rig):
    """The pool holds 40 pages; the requests below need 76 in total, at most 38 at a time."""
    V = rig.cfg["vocab"]
    free0 = rig.engine.num_free_blocks()
    for rnd in range(4):
        pr = {"x": toks(300, V, 20 + rnd), "y": toks(290, V, 30 + rnd)}
        rig.check(pr, [[("x", 150), ("y", 7)], [("x", 149), ("y", 282)], [("x", 1), ("y", 1)]])
        assert rig.engine.num_free_blocks() == free0


def test_pool_exhaustion_is_refused_and_changes_nothing(rig):
    V = rig.cfg["vocab"]
    a, b = rig.engine.open_request(), rig.engine.open_request()
    rig.engine.step_forced([(a, toks(400, V, 40), [])])
    free = rig.engine.num_free_blocks()
    with pytest.raises(rig.eng.NvcError):
        rig.engine.step_forced([(b, toks(300, V, 41), [])])
    assert rig.engine.num_free_blocks() == free
    p = toks(100, V, 42)
    lg = rig.engine.step_forced([(b, p, [99])])
    assert rig.rel_err(lg[:1], rig.want(p)[99:100])[0] < rig.tol
    rig.engine.close_request(a)
    rig.engine.close_request(b)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(dtype):
    r = Rig(cfg_b(), dtype, blocks=12, seed=3)
    try:
        V = r.cfg["vocab"]
        pr = {"a": toks(50, V, 1), "b": toks(19, V, 2)}
        r.check(pr, [[("a", 20), ("b", 19)], [("a", 2)], [("a", 27)], [("a", 1)]])
    finally:
        r.close()


def cfg_c():
    """Every latent pads to 128 numbers, the width at which long prompt portions of the bf16 mode run on the tcgen05
    paged-prefill kernel (as multi-query attention over the latent rows); head counts that divide nothing."""
    return K.make_config(vocab=160, width=128, layers=[
        {"type": "latent_attention", "mixer": K.mixer_cfg(3, 32, 16, 128, 48, 0.2), "mlp": K.dense_cfg(96)},
        {"type": "latent_attention", "mixer": K.mixer_cfg(5, 16, 24, 100, 32, 0.3), "mlp": None},
    ], loop={"start": 0, "stop": 2, "times": 2})


def cfg_d():
    """Experts wide enough (128 and more after padding) for the grouped tcgen05 products of the bf16 mode; every expert is
    chosen, so that no rounding of a router's input can flip a choice."""
    return K.make_config(vocab=200, width=192, layers=[
        {"type": "latent_attention", "mixer": K.mixer_cfg(2, 32, 32, 64, 32, 0.2), "mlp": K.moe_cfg(3, 3, 136, 1.2, 72)},
        {"type": "latent_attention", "mixer": K.mixer_cfg(3, 16, 16, 48, 24, 0.25), "mlp": K.moe_cfg(2, 2, 200, 0.8, 0)},
    ], loop=None)


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_wide_experts(dtype):
    r = Rig(cfg_d(), dtype, blocks=40, seed=21)
    try:
        V = r.cfg["vocab"]
        pr = {"a": toks(300, V, 70), "b": toks(45, V, 71), "c": toks(2, V, 72)}
        r.check(pr, [[("a", 200), ("b", 1)], [("b", 1), ("a", 99), ("c", 2)], [("a", 1), ("b", 43)]])
    finally:
        r.close()


@pytest.mark.parametrize("flash", ["1", "0"])
def test_long_portions_beside_decoded_tokens(monkeypatch, flash):
    """Portions of 64 tokens and more - whole prompts, behind a cached prefix that ends inside a page, beside one-token
    sequences of the same step - against the oracle, with the tcgen05 route on and off (the two must agree with the
    oracle alike: which kernel computed a position depends on the schedule)."""
    monkeypatch.setenv("NVC_KARUZEN_FLASH", flash)
    r = Rig(cfg_c(), "bfloat16", blocks=48, seed=12)
    try:
        V = r.cfg["vocab"]
        pr = {"a": toks(333, V, 60), "b": toks(131, V, 61), "c": toks(70, V, 62), "d": toks(5, V, 63)}
        sched = [[("a", 129), ("d", 1)], [("d", 1), ("a", 64), ("b", 77)], [("d", 1), ("a", 1), ("b", 3), ("c", 70)],
                 [("d", 1), ("b", 51), ("a", 139)], [("d", 1)]]
        assert all(sum(n for s in sched for k, n in s if k == name) == len(p) for name, p in pr.items())
        r.check(pr, sched)
        # a whole prompt in one portion, then the same prompt cut after nine tokens (prefix shorter than a page)
        r.check({"w": toks(200, V, 64)}, [[("w", 200)]])
        r.check({"w": toks(200, V, 64)}, [[("w", 9)], [("w", 191)]])
    finally:
        r.close()


@pytest.mark.parametrize("dtype,chunked", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_greedy_generation_through_the_scheduler(dtype, chunked):
    """LLMEngine.generate: the engine's own admission, paged prefill, graph-captured decode steps.  Every generated token
    must be the oracle's argmax on the same prefix (fp32) or within the bf16 error of its best logit."""
    r = Rig(cfg_a(all_experts=dtype == "bfloat16"), dtype, blocks=24, seed=5, chunked=chunked)
    try:
        V = r.cfg["vocab"]
        prompts = [toks(n, V, 50 + n) for n in (5, 33, 16)]
        outs = r.engine.generate(prompts, r.eng.SamplingParams(1.0, 12, True))
        assert len(outs) == 3
        for p, o in zip(prompts, outs):
            assert len(o.token_ids) == 12
            lg = r.want(p + o.token_ids[:-1])
            for i, t in enumerate(o.token_ids):
                row = lg[len(p) - 1 + i]
                assert row.max() - row[t] <= (1e-3 if dtype == "float32" else 0.25), f"token {i}"
        assert r.engine.num_free_blocks() == 24
    finally:
        r.close()


def write_model_dir(path, cfg, weights):
    """config.json + model.safetensors (bf16) the way a checkpoint of this design is stored."""
    import json
    import struct
    header, blobs, at = {}, [], 0
    for name, t in weights.items():
        raw = t.bfloat16().contiguous().view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    hj += b" " * (-len(hj) % 8)
    with open(path / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)) + hj + b"".join(blobs))
    (path / "config.json").write_text(json.dumps(cfg))


def test_command_line_tools_on_a_checkpoint_directory(tmp_path):
    """bin/trace_run and bin/generate: registry by config.json, native safetensors loader, the engine underneath."""
    import json
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cfg = cfg_a()
    w = K.make_weights(cfg, 9)
    oracle = K.KaruzenOracle(cfg, w)
    write_model_dir(tmp_path, cfg, w)
    V = cfg["vocab"]
    pa, pb = toks(41, V, 1), toks(9, V, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": pa[:30], "want": [0, 29]}, {"id": "b", "tokens": pb[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": pb[2:], "want": [6]}, {"id": "a", "tokens": pa[30:31], "want": [0]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "a", "tokens": pa[31:], "want": [9]}, {"id": "b", "tokens": pb, "want": [8]}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    r = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(tmp_path), "--dtype", "float32", "--out", str(out),
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    la, lb = oracle.forward(pa).numpy(), oracle.forward(pb).numpy()
    want = {0: np.stack([la[0], la[29]]), 1: np.stack([lb[8], la[30]]), 2: np.stack([la[40], lb[8]])}
    for n, wv in want.items():
        got = np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, V)
        assert got.shape == wv.shape and Rig.rel_err(got, wv).max() < 1e-4, f"step {n}"
    g = subprocess.run([sys.executable, os.path.join(root, "bin", "generate"), "--model", str(tmp_path), "--dtype", "float32", "--prompt-ids",
                        ",".join(map(str, pb)) + ";" + ",".join(map(str, pa[:5])), "--max-tokens", "6", "--block-size", "16"],
                       capture_output=True, text=True, timeout=600)
    assert g.returncode == 0, g.stderr[-2000:]
    lines = [json.loads(ln) for ln in g.stdout.splitlines() if ln.startswith("{")]
    assert [ln["prompt"] for ln in lines] == [pb, pa[:5]]
    for ln in lines:
        lg = oracle.forward(ln["prompt"] + ln["tokens"][:-1]).numpy()
        for i, t in enumerate(ln["tokens"]):
            row = lg[len(ln["prompt"]) - 1 + i]
            assert row.max() - row[t] <= 1e-3
