"""Host side of the Karuzen family, no GPU: the registry's configuration parser, the order of layer runs, the plain
oracle's own consistency (whole prompt = portions = token by token) and the caller-driven engine API's refusals."""
import ctypes as C
import importlib
import json

import numpy as np
import pytest
import torch

from oracle import karuzen_oracle as K


@pytest.fixture(scope="module")
def lib(nvc):
    return nvc.lib()


def parse(lib, cfg):
    h = C.c_void_p()
    st = lib.nvc_model_config_from_json(json.dumps(cfg).encode(), C.byref(h))
    return st, h


def small_cfg(**kw):
    layers = [{"type": "latent_attention", "mixer": K.mixer_cfg(2, 8, 16, 24, 8, 0.3), "mlp": m}
              for m in (K.dense_cfg(32), K.moe_cfg(4, 2, 16, 1.5, 24), None, K.moe_cfg(3, 1, 8, 0.5, 0), K.dense_cfg(16))]
    return K.make_config(vocab=50, width=40, layers=layers, **kw)


@pytest.mark.parametrize("loop", [None, {"start": 0, "stop": 2, "times": 3}, {"start": 1, "stop": 4, "times": 2},
                                  {"start": 2, "stop": 5, "times": 1}, {"start": 3, "stop": 3, "times": 4}])
def test_layer_runs_follow_the_loop(lib, loop):
    cfg = small_cfg(loop=loop)
    st, h = parse(lib, cfg)
    assert st == 0, lib.nvc_model_config_last_error().decode()
    assert lib.nvc_model_config_architecture(h).decode() == "Karuzen" and lib.nvc_model_config_vocab(h) == 50
    a, b, c = (np.zeros(64, np.int32) for _ in range(3))
    n = lib.nvc_model_config_layer_runs(h, a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), c.ctypes.data_as(C.c_void_p), 64)
    lib.nvc_model_config_free(h)
    want = K.layer_runs(cfg)
    assert n == len(want)
    assert [(int(a[i]), int(b[i]), bool(c[i])) for i in range(n)] == want


def test_bad_configurations_are_refused(lib):
    def bad(mut):
        cfg = small_cfg(loop={"start": 0, "stop": 2, "times": 2})
        mut(cfg)
        st, h = parse(lib, cfg)
        if st == 0:
            lib.nvc_model_config_free(h)
        return st != 0 and len(lib.nvc_model_config_last_error()) > 0

    assert bad(lambda c: c.update(architecture="Nonesuch"))
    assert bad(lambda c: c.pop("width"))
    assert bad(lambda c: c["layers"][0].update(type="window_attention"))
    assert bad(lambda c: c["layers"][0]["mixer"].pop("kv_rank"))
    assert bad(lambda c: c["layers"][1]["mlp"]["router"].update(top=5))
    assert bad(lambda c: c["layers"][0]["mlp"].update(kind="conv"))
    assert bad(lambda c: c["loop"].update(stop=9))
    assert bad(lambda c: c["loop"].update(start=3))
    assert bad(lambda c: c["norm"].pop("eps"))
    assert bad(lambda c: c.update(layers=[]))


def test_oracle_is_schedule_independent():
    cfg = small_cfg(loop={"start": 1, "stop": 3, "times": 2})
    o = K.KaruzenOracle(cfg, K.make_weights(cfg, 1))
    toks = torch.randint(0, 50, (23,), generator=torch.Generator().manual_seed(2)).tolist()
    whole = o.forward(toks)
    cache = o.new_cache()
    parts = torch.cat([o.forward(toks[:9], cache), o.forward(toks[9:11], cache)] + [o.forward([t], cache) for t in toks[11:]])
    assert torch.allclose(whole, parts, rtol=1e-4, atol=1e-4)
    # the causal bound: a later token does not change earlier logits
    assert torch.allclose(o.forward(toks[:10]), whole[:10], rtol=1e-4, atol=1e-4)


def test_absorbed_form_equals_per_head_keys_and_values():
    """What the CUDA path computes - queries carried through uk into the latent space, one shared row per token, uv
    applied after the softmax - equals attention over per-head keys and values rebuilt from the latents."""
    g = torch.Generator().manual_seed(3)
    m = K.mixer_cfg(3, 8, 12, 20, 16, 0.4)
    W = 24
    p = {"dq": torch.randn(16, W, generator=g), "dq.norm": torch.ones(16), "uq": torch.randn(24, 16, generator=g),
         "dkv": torch.randn(20, W, generator=g), "dkv.norm": torch.ones(20), "uk": torch.randn(24, 20, generator=g),
         "uv": torch.randn(36, 20, generator=g), "o": torch.randn(W, 36, generator=g)}
    h = torch.randn(7, W, generator=g)
    want, c = K.latent_attention(h, p, m, 1e-5)
    cq, _ = K.latents(h, p["dq"], p["dq.norm"], p["dkv"], p["dkv.norm"], 1e-5)
    q = (cq @ p["uq"].T).view(7, 3, 8)
    qabs = torch.einsum("ihd,hdc->ihc", q, p["uk"].view(3, 8, 20))
    s = torch.einsum("ihc,jc->hij", qabs, c) * m["scale"]
    s = s.masked_fill(torch.arange(7).view(1, 1, 7) > torch.arange(7).view(1, 7, 1), float("-inf"))
    olat = torch.einsum("hij,jc->ihc", torch.softmax(s, -1), c)
    got = torch.einsum("ihc,hvc->ihv", olat, p["uv"].view(3, 12, 20)).reshape(7, 36) @ p["o"].T
    assert torch.allclose(got, want, rtol=1e-4, atol=1e-4)


def test_caller_driven_requests_need_chunked_mode_and_a_runner(nvc):
    eng = importlib.import_module("nano-vllm-candle_b200.engine")
    e = eng.LLMEngine(eng.Scheduler(eng.SchedulerConfig(4, 256, -1, 8, 16)), eng.DummyModelRunner(), greedy=True)
    with pytest.raises(eng.NvcError):
        e.open_request()
    e.close()
    e = eng.LLMEngine(eng.Scheduler(eng.SchedulerConfig(4, 256, -1, 8, 16, enable_chunked_prefill=True)), eng.DummyModelRunner(),
                      greedy=True)
    sid = e.open_request()
    so = C.c_void_p()
    ids, counts, toks = np.array([sid], np.int64), np.array([2], np.int32), np.array([1, 2], np.int32)
    st = e.l.nvc_engine_step_forced(e.h, 1, ids.ctypes.data_as(C.c_void_p), counts.ctypes.data_as(C.c_void_p),
                                    toks.ctypes.data_as(C.c_void_p), None, None, None)
    assert st != 0                       # no model runner behind this engine
    assert e.num_free_blocks() == 8
    e.close_request(sid)
    with pytest.raises(eng.NvcError):
        e.close_request(sid)
    e.close()
