"""Ranilix through the runner and the engine: logits of every position against the plain fp32 oracle, whatever the
schedule - whole prompts, token-by-token decoding, portions down to two tokens, mixed batches, reused pages and state
slots - plus greedy generation through LLMEngine's own scheduler.  Small configurations whose sizes differ from one
another (head counts, key / value sizes, rotated parts, windows, decays), layers without feed-forward, blending and
non-blending attention layers, a model that starts with a parallel layer."""
import importlib

import numpy as np
import pytest
import torch

from oracle import ranilix_oracle as R

pytestmark = pytest.mark.gpu
BLOCK = 16


def cfg_a():
    """attention (provides the blended values) / parallel / attention (blends) / parallel without feed-forward."""
    return R.make_config(vocab=200, width=96, layers=[
        R.with_mlp(R.attention_cfg(4, 2, 32, 24, window=12, rot_dims=16, scale=0.2), 160),
        R.with_mlp(R.parallel_cfg(4, 2, 32, 40, rot_dims=8, r_heads=3, r_dim=16, r_vdim=24, r_rot_dims=16, decay=(0.9, 0.97, 0.995)), 96),
        R.with_mlp(R.attention_cfg(2, 1, 48, 48, window=21, rot_dims=48, rot_base=300.0, scale=0.15), 64),
        R.with_mlp(R.parallel_cfg(3, 3, 16, 16, rot_dims=0, r_heads=1, r_dim=40, r_vdim=72, r_rot_dims=20, decay=(0.999,), left_scale=0.7, right_scale=1.3), None),
    ])


def cfg_b():
    """Starts with a parallel layer; an attention layer that does not blend between two that do; a window of one token;
    an attention layer without a window; a width and a vocabulary that are multiples of nothing."""
    return R.make_config(vocab=203, width=100, embedding_scale=1.0, eps=1e-3, layers=[
        R.with_mlp(R.parallel_cfg(2, 1, 24, 8, rot_dims=24, r_heads=2, r_dim=8, r_vdim=40, r_rot_dims=0, decay=(0.5, 1.0)), 72),
        R.with_mlp(R.attention_cfg(5, 5, 8, 16, window=1, rot_dims=4, scale=0.4), None),
        R.with_mlp(R.attention_cfg(1, 1, 64, 80, window=None, rot_dims=32, scale=0.1, v_mix=False), 40),
        R.with_mlp(R.attention_cfg(5, 1, 16, 80, window=40, rot_dims=0, scale=0.3), 56),
    ])


def cfg_c():
    """Head sizes that are multiples of 16 (the tensor-pipe attention of the bf16 mode), unequal key and value sizes."""
    return R.make_config(vocab=160, width=128, layers=[
        R.with_mlp(R.attention_cfg(4, 2, 64, 32, window=50, rot_dims=32, scale=0.125), 192),
        R.with_mlp(R.parallel_cfg(4, 4, 32, 128, rot_dims=16, scale=0.17, r_heads=2, r_dim=32, r_vdim=64, r_rot_dims=32, decay=(0.98, 0.9995)), 128),
        R.with_mlp(R.attention_cfg(8, 2, 16, 32, window=129, rot_dims=16, scale=0.25), None),
    ])


def cfg_d():
    """Parallel layers whose causal half has keys and values of 128 numbers: in the bf16 mode its long prompt portions run on the
    tcgen05 paged-prefill kernel; one of them shares key heads between query heads, and both weights differ from 1."""
    return R.make_config(vocab=180, width=192, layers=[
        R.with_mlp(R.parallel_cfg(2, 1, 128, 128, rot_dims=64, scale=0.09, left_scale=1.4, r_heads=2, r_dim=16, r_vdim=32, r_rot_dims=8, decay=(0.9, 0.99), right_scale=0.7), 128),
        R.with_mlp(R.attention_cfg(2, 2, 32, 32, window=70, rot_dims=16, scale=0.2), None),
        R.with_mlp(R.parallel_cfg(3, 3, 128, 128, rot_dims=0, scale=0.08, left_scale=0.6, r_heads=1, r_dim=24, r_vdim=40, r_rot_dims=24, decay=(0.995,), right_scale=1.2), 96),
    ])


class Rig:
    def __init__(self, cfg, dtype, blocks=40, seed=0, chunked=True, seqs=4, weights=None):
        self.eng = importlib.import_module("nano-vllm-candle_b200.engine")
        self.cfg, self.dtype = cfg, dtype
        self.w = weights if weights is not None else R.make_weights(cfg, seed)
        self.oracle = R.RanilixOracle(cfg, self.w)
        self.ctx = self.eng.DeviceContext(0)
        T = blocks * BLOCK
        self.blocks = blocks
        self.runner = self.eng.ModelRunner.from_config(self.ctx, cfg, self.w.items(), num_kvcache_blocks=blocks, kvcache_block_size=BLOCK,
                                                       max_num_seqs=seqs, max_num_batched_tokens=T, max_model_len=T, dtype=dtype,
                                                       max_logit_rows=T)
        sc = self.eng.SchedulerConfig(max_num_seqs=seqs, max_num_batched_tokens=T, eos=-1, num_kvcache_blocks=blocks,
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
    r = Rig(cfg_a(), request.param)
    yield r
    r.close()


def test_whole_prompts_and_first_tokens(rig):
    V = rig.cfg["vocab"]
    rig.check({"one": toks(1, V, 1)}, [[("one", 1)]])
    rig.check({"two": toks(2, V, 2)}, [[("two", 2)]])
    rig.check({"p": toks(83, V, 2)}, [[("p", 83)]])
    rig.check({"page": toks(2 * BLOCK, V, 3)}, [[("page", 2 * BLOCK)]])


def test_residual_stream_after_every_layer(rig):
    p = toks(21, rig.cfg["vocab"], 4)
    tap = rig.runner.tap_residual(len(p))
    sid = rig.engine.open_request()
    rig.engine.step_forced([(sid, p, [0])])
    rig.engine.close_request(sid)
    res = []
    rig.oracle.forward(p, residuals=res)
    assert tap.shape[0] == len(res) == 4
    for k, want in enumerate(res):
        assert np.abs(tap[k] - want.numpy()).max() < (2e-4 if rig.dtype == "float32" else 0.3), f"layer {k}"


def test_prefill_then_token_by_token(rig):
    p = toks(70, rig.cfg["vocab"], 5)
    rig.check({"d": p}, [[("d", 30)]] + [[("d", 1)]] * 40)       # both windows (12, 21) pass over decoded tokens
    rig.check({"d": p}, [[("d", 1)]] * 70)                       # decoding from the very first token, across page borders


def test_portions_of_many_sizes(rig):
    p = toks(121, rig.cfg["vocab"], 6)
    sizes = [2, 14, 16, 1, 17, 2, 31, 3, 33, 2]        # cuts before, at and after page borders and inside windows
    assert sum(sizes) == 121
    rig.check({"c": p}, [[("c", n)] for n in sizes])
    rig.check({"c": p}, [[("c", 2)]] * 60 + [[("c", 1)]])


def test_long_decoding(rig):
    p = toks(300, rig.cfg["vocab"], 7)
    rig.check({"l": p}, [[("l", 5)]] + [[("l", 1)]] * 295)


def test_mixed_batches_equal_each_request_alone(rig):
    V = rig.cfg["vocab"]
    pr = {"a": toks(90, V, 8), "b": toks(37, V, 9), "c": toks(3, V, 10), "d": toks(64, V, 11)}
    sched = [[("a", 40), ("b", 2)], [("a", 1), ("b", 20), ("c", 1)], [("a", 1), ("c", 1), ("d", 64)], [("a", 17), ("b", 1), ("c", 1)],
             [("a", 1), ("b", 14)]] + [[("a", 1)]] * 30
    assert all(sum(n for s in sched for k, n in s if k == name) == len(p) for name, p in pr.items())
    rig.check(pr, sched)


def test_a_request_left_out_of_steps_goes_on_later(rig):
    V = rig.cfg["vocab"]
    pr = {"a": toks(50, V, 12), "b": toks(45, V, 13)}
    rig.check(pr, [[("a", 10), ("b", 5)], [("b", 20)], [("b", 1)], [("a", 1), ("b", 1)], [("b", 18)], [("a", 39)]])


def test_steps_without_wanted_logits(rig):
    """Steps that ask for no logits: single tokens go through the captured decode step (the state slots ride in its one
    upload), portions through the mixed step; the next wanted position must not notice."""
    V = rig.cfg["vocab"]
    pa, pb = toks(60, V, 14), toks(45, V, 15)
    a, b = rig.engine.open_request(), rig.engine.open_request()
    rig.engine.step_forced([(a, pa[:20], []), (b, pb[:3], [])])
    for i in range(30):
        rig.engine.step_forced([(b, pb[3 + i:4 + i], []), (a, pa[20 + i:21 + i], [])])      # decode steps, nothing wanted
    rig.engine.step_forced([(a, pa[50:59], [])])
    lg = rig.engine.step_forced([(a, pa[59:], [0]), (b, pb[33:], [0, 11])])
    wa, wb = rig.want(pa), rig.want(pb)
    err = rig.rel_err(lg, np.stack([wa[59], wb[33], wb[44]]))
    assert err.max() < rig.tol, err
    rig.engine.close_request(a)
    rig.engine.close_request(b)


def test_pages_and_state_slots_are_freed_and_used_again(rig):
    """The pool holds 40 pages and four state slots; the requests below need 76 pages in total, at most 38 at a time, and
    every round takes state slots that the round before has left full."""
    V = rig.cfg["vocab"]
    free0 = rig.engine.num_free_blocks()
    for rnd in range(4):
        pr = {"x": toks(300, V, 20 + rnd), "y": toks(290, V, 30 + rnd)}
        rig.check(pr, [[("x", 150), ("y", 7)], [("x", 149), ("y", 282)], [("x", 1), ("y", 1)]])
        assert rig.engine.num_free_blocks() == free0
    # all four slots live at once, closed in another order than opened, then taken again
    for rnd in range(2):
        pr = {k: toks(20 + 3 * i, V, 40 + 10 * rnd + i) for i, k in enumerate("pqrs")}
        rig.check(pr, [[("p", 5), ("q", 23)], [("r", 10), ("p", 1), ("s", 2)], [("s", 27), ("p", 14), ("r", 16)]])


def test_a_fifth_live_request_is_refused_and_changes_nothing(rig):
    V = rig.cfg["vocab"]
    ids = [rig.engine.open_request() for _ in range(5)]
    rig.engine.step_forced([(i, toks(3, V, 50 + k), []) for k, i in enumerate(ids[:4])])
    free = rig.engine.num_free_blocks()
    with pytest.raises(rig.eng.NvcError):
        rig.engine.step_forced([(ids[4], toks(3, V, 60), [])])
    assert rig.engine.num_free_blocks() == free
    rig.engine.close_request(ids[0])
    p = toks(30, V, 61)
    lg = rig.engine.step_forced([(ids[4], p, [29])])
    assert rig.rel_err(lg[:1], rig.want(p)[29:30])[0] < rig.tol
    for i in ids[1:]:
        rig.engine.close_request(i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_other_sizes(dtype):
    r = Rig(cfg_b(), dtype, blocks=12, seed=3)
    try:
        V = r.cfg["vocab"]
        pr = {"a": toks(100, V, 1), "b": toks(19, V, 2)}
        r.check(pr, [[("a", 20), ("b", 19)], [("a", 2)], [("a", 27)], [("a", 1)]] + [[("a", 1)]] * 50)
    finally:
        r.close()


@pytest.mark.parametrize("dtype", ["bfloat16", "float32"])
def test_head_sizes_of_the_tensor_pipe_attention(dtype):
    r = Rig(cfg_c(), dtype, blocks=48, seed=12)
    try:
        V = r.cfg["vocab"]
        pr = {"a": toks(333, V, 60), "b": toks(131, V, 61), "c": toks(70, V, 62), "d": toks(5, V, 63)}
        sched = [[("a", 129), ("d", 1)], [("d", 1), ("a", 64), ("b", 77)], [("d", 1), ("a", 1), ("b", 3), ("c", 70)],
                 [("d", 1), ("b", 51), ("a", 139)], [("d", 1)]]
        assert all(sum(n for s in sched for k, n in s if k == name) == len(p) for name, p in pr.items())
        r.check(pr, sched)
        r.check({"w": toks(200, V, 64)}, [[("w", 9)], [("w", 191)]])
        r.check({"w": toks(200, V, 64)}, [[("w", 140)]] + [[("w", 1)]] * 60)
    finally:
        r.close()


@pytest.mark.parametrize("flash", ["1", "0"])
def test_long_portions_of_the_causal_half_beside_decoded_tokens(monkeypatch, flash):
    """Portions of 64 tokens and more - whole prompts, behind a cached prefix that ends inside a page, beside one-token
    sequences of the same step - with the tcgen05 route of the causal half on and off: which kernel computed a position depends
    on the schedule, so both must agree with the oracle alike."""
    monkeypatch.setenv("NVC_RANILIX_FLASH", flash)
    r = Rig(cfg_d(), "bfloat16", blocks=48, seed=12)
    try:
        V = r.cfg["vocab"]
        pr = {"a": toks(333, V, 60), "b": toks(131, V, 61), "c": toks(70, V, 62), "d": toks(5, V, 63)}
        sched = [[("a", 129), ("d", 1)], [("d", 1), ("a", 64), ("b", 77)], [("d", 1), ("a", 1), ("b", 3), ("c", 70)],
                 [("d", 1), ("b", 51), ("a", 139)], [("d", 1)]]
        assert all(sum(n for s in sched for k, n in s if k == name) == len(p) for name, p in pr.items())
        r.check(pr, sched)
        r.check({"w": toks(200, V, 64)}, [[("w", 200)]])
        r.check({"w": toks(200, V, 64)}, [[("w", 9)], [("w", 191)]])
        r.check({"w": toks(200, V, 64)}, [[("w", 150)]] + [[("w", 1)]] * 50)
    finally:
        r.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("gap", [11, 12, 13])
def test_one_token_before_and_after_the_window_edge(dtype, gap):
    """One attention layer with a window of 12 (the position itself and the 11 before it): another token is planted `gap`
    positions before the end.  Inside the window it moves the last logits; one position outside, it moves nothing.  The
    runner must agree with the oracle for a whole prompt, for a portion that starts between the two and for decoding."""
    cfg = R.make_config(vocab=60, width=64, layers=[R.with_mlp(R.attention_cfg(2, 1, 32, 32, window=12, rot_dims=16, scale=0.5, v_mix=False), None)])
    w = R.make_weights(cfg, 30)
    w["l0.mix.sink"] = torch.full((2,), -30.0)                 # no sink weight: the window's keys share all of it
    r = Rig(cfg, dtype, blocks=8, weights=w)
    try:
        n = 40
        p = [3 + (i % 3) for i in range(n)]
        p[n - 1 - gap] = 7
        r.check({"w": p}, [[("w", n)]])
        r.check({"w": p}, [[("w", n - 5)], [("w", 5)]])
        r.check({"w": p}, [[("w", n - 20)]] + [[("w", 1)]] * 20)
        q = list(p)
        q[n - 1 - gap] = 4
        moved = Rig.rel_err(r.want(p)[-1:], r.want(q)[-1:])[0]
        assert moved > 0.01 if gap < 12 else moved < 1e-6
        got_p, got_q = r.replay({"w": p}, [[("w", n - 20)]] + [[("w", 1)]] * 20)["w"], r.replay({"w": q}, [[("w", n - 20)]] + [[("w", 1)]] * 20)["w"]
        moved = Rig.rel_err(got_p[-1:], got_q[-1:])[0]
        assert moved > 0.01 if gap < 12 else moved < 1e-6
    finally:
        r.close()


@pytest.mark.parametrize("dtype,chunked", [("float32", False), ("float32", True), ("bfloat16", True)])
def test_greedy_generation_through_the_scheduler(dtype, chunked):
    """LLMEngine.generate: the engine's own admission, state slots, paged prefill, graph-captured decode steps.  Every
    generated token must be the oracle's argmax on the same prefix (fp32) or within the bf16 error of its best logit."""
    r = Rig(cfg_a(), dtype, blocks=24, seed=5, chunked=chunked)
    try:
        V = r.cfg["vocab"]
        prompts = [toks(n, V, 50 + n) for n in (5, 33, 16, 2, 40, 9)]      # more requests than state slots
        outs = r.engine.generate(prompts, r.eng.SamplingParams(1.0, 12, True))
        assert len(outs) == 6
        for p, o in zip(prompts, outs):
            assert len(o.token_ids) == 12
            lg = r.want(p + o.token_ids[:-1])
            for i, t in enumerate(o.token_ids):
                row = lg[len(p) - 1 + i]
                assert row.max() - row[t] <= (1e-3 if dtype == "float32" else 0.25), f"token {i}"
        assert r.engine.num_free_blocks() == 24
    finally:
        r.close()


def test_prefix_caching_is_refused_for_a_model_with_recurrent_state():
    r = Rig(cfg_a(), "float32", blocks=8)
    try:
        sc = r.eng.SchedulerConfig(max_num_seqs=4, max_num_batched_tokens=8 * BLOCK, eos=-1, num_kvcache_blocks=8, kvcache_block_size=BLOCK,
                                   enable_prefix_caching=True, enable_chunked_prefill=True, max_model_len=8 * BLOCK)
        with pytest.raises(Exception):
            r.eng.LLMEngine(r.eng.Scheduler(sc), r.runner, greedy=True)
        assert r.runner.num_state_slots() == 4
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
    w = R.make_weights(cfg, 9)
    oracle = R.RanilixOracle(cfg, w)
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
