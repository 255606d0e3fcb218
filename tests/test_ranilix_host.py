"""Host side of the Ranilix family, no GPU: the registry's configuration parser and the plain oracle's own consistency
(whole prompt = portions = token by token; the window, the sink and the recurrence do what their formulas say)."""
import ctypes as C
import json

import pytest
import torch

from oracle import ranilix_oracle as R


@pytest.fixture(scope="module")
def lib(nvc):
    return nvc.lib()


def parse(lib, cfg):
    h = C.c_void_p()
    st = lib.nvc_model_config_from_json(json.dumps(cfg).encode(), C.byref(h))
    return st, h


def small_cfg():
    return R.make_config(vocab=50, width=40, layers=[
        R.with_mlp(R.attention_cfg(2, 1, 8, 12, window=5, rot_dims=4), 32),
        R.with_mlp(R.parallel_cfg(2, 2, 8, 16, rot_dims=8, r_heads=2, r_dim=4, r_vdim=6, r_rot_dims=4, decay=(0.8, 0.95)), None),
        R.with_mlp(R.attention_cfg(3, 1, 4, 12, window=None, rot_dims=0), 16),
    ])


def test_configuration_is_taken_by_the_registry(lib):
    st, h = parse(lib, small_cfg())
    assert st == 0, lib.nvc_model_config_last_error().decode()
    assert lib.nvc_model_config_architecture(h).decode() == "Ranilix" and lib.nvc_model_config_vocab(h) == 50
    assert lib.nvc_model_config_layer_runs(h, None, None, None, 0) == 3
    lib.nvc_model_config_free(h)


def test_bad_configurations_are_refused(lib):
    def bad(mut):
        cfg = small_cfg()
        mut(cfg)
        st, h = parse(lib, cfg)
        if st == 0:
            lib.nvc_model_config_free(h)
        return st != 0 and len(lib.nvc_model_config_last_error()) > 0

    assert bad(lambda c: c.pop("width"))
    assert bad(lambda c: c["norm"].pop("eps"))
    assert bad(lambda c: c.update(layers=[]))
    assert bad(lambda c: c["layers"][0].update(type="convolution"))
    assert bad(lambda c: c["layers"][0]["mixer"].pop("vdim"))
    assert bad(lambda c: c["layers"][0]["mixer"].update(kv_heads=3))            # heads not a multiple
    assert bad(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=5))         # odd
    assert bad(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=10))        # above dim
    assert bad(lambda c: c["layers"][0]["mixer"]["mask"].update(size=0))
    assert bad(lambda c: c["layers"][1]["mixer"]["right"].update(decay=[0.5]))  # one per head
    assert bad(lambda c: c["layers"][1]["mixer"].pop("left_scale"))
    assert bad(lambda c: c["layers"][1]["mixer"].pop("right"))
    assert bad(lambda c: c["layers"][0]["mlp"].update(kind="moe"))
    assert bad(lambda c: c["layers"][2]["mixer"].update(vdim=5))                # blending layers disagree on the value width


def test_oracle_is_schedule_independent():
    cfg = small_cfg()
    o = R.RanilixOracle(cfg, R.make_weights(cfg, 1))
    toks = torch.randint(0, 50, (23,), generator=torch.Generator().manual_seed(2)).tolist()
    whole = o.forward(toks)
    cache = o.new_cache()
    parts = torch.cat([o.forward(toks[:9], cache), o.forward(toks[9:11], cache)] + [o.forward([t], cache) for t in toks[11:]])
    assert torch.allclose(whole, parts, rtol=1e-4, atol=1e-4)
    assert torch.allclose(o.forward(toks[:10]), whole[:10], rtol=1e-4, atol=1e-4)     # causal


def test_oracle_window_and_sink():
    g = torch.Generator().manual_seed(3)
    q, k, v = torch.randn(1, 1, 4, generator=g), torch.randn(10, 1, 4, generator=g), torch.randn(10, 1, 3, generator=g)
    pos = torch.tensor([9])
    full = R.softmax_attention(q, k, v, 1.0, pos)
    win = R.softmax_attention(q, k, v, 1.0, pos, window=4)
    tail = R.softmax_attention(q, k[6:], v[6:], 1.0, torch.tensor([3]))
    assert torch.allclose(win, tail, atol=1e-6) and not torch.allclose(win, full, atol=1e-3)
    s = (q[0, 0] @ k[:, 0].T)
    sink = torch.tensor([0.7])
    want = (torch.exp(s) / (torch.exp(s).sum() + torch.exp(sink))) @ v[:, 0]
    assert torch.allclose(R.softmax_attention(q, k, v, 1.0, pos, None, sink)[0], want, atol=1e-6)


def test_oracle_retention_closed_form():
    """o_t = sum_{j <= t} decay^(t - j) (q_t . k_j) v_j with k scaled by dim^-1/2."""
    m = {"heads": 1, "dim": 4, "vdim": 3, "decay": [0.9], "rot": {"dims": 0, "base": 1.0}}
    g = torch.Generator().manual_seed(4)
    W = 6
    p = {n: torch.randn(r, W, generator=g) for n, r in (("q", 4), ("k", 4), ("v", 3), ("g", 3))}
    p["o"] = torch.eye(3)
    h = torch.randn(5, W, generator=g)
    out, S = R.retention(h, p, m, 1e-6, 0)
    q, k, v = h @ p["q"].T, (h @ p["k"].T) * 0.5, h @ p["v"].T
    o = torch.stack([sum(0.9 ** (t - j) * (q[t] @ k[j]) * v[j] for j in range(t + 1)) for t in range(5)])
    gate = h @ p["g"].T
    want = R.rms_norm(o, None, 1e-6) * gate * torch.sigmoid(gate)
    assert torch.allclose(out, want, atol=1e-5)
    out2, _ = R.retention(h[3:], p, m, 1e-6, 3, R.retention(h[:3], p, m, 1e-6, 0)[1])
    assert torch.allclose(out2, want[3:], atol=1e-5)
