"""Plain fp32 restatement of the Karuzen design, one function per mechanism, slow on purpose.

Notation: W (width), V (vocab), T (tokens of one sequence).  Linear weights are [out, in] and act as
y = W x.  A layer is parallel: h = dyt(x); x <- x + mixer(h) + ff(h).  The looped block [start, stop)
runs `times` passes with the same weights; before every pass but the first the embedding output is
added to x.  Everything here is float32 torch on the CPU; nothing is shared with the CUDA path.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def dyt(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, alpha: torch.Tensor) -> torch.Tensor:
    """Dynamic Tanh: tanh(alpha x) w + b, no statistics of x."""
    return torch.tanh(alpha * x) * w + b


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def latents(h, dq, dq_norm, dkv, dkv_norm, eps):
    """(query latent, key/value latent) of every token: both RMS-normed low-rank projections."""
    return rms_norm(h @ dq.T, dq_norm, eps), rms_norm(h @ dkv.T, dkv_norm, eps)


def latent_attention_scores(q, k, scale):
    """[heads, Tq, Tk] raw scores of per-head queries [Tq, heads, d] against keys [Tk, heads, d]."""
    return torch.einsum("ihd,jhd->hij", q, k) * scale


def latent_attention(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float,
                     c_prefix: Optional[torch.Tensor] = None):
    """Causal latent attention over one sequence.  h: [T, W] inputs of the NEW tokens; c_prefix: latents of
    the tokens before them (what a cache holds).  Keys and values are rebuilt from the latents, head by
    head.  Returns (output [T, W], all latents [T_prefix + T, kv_rank])."""
    T, H, d, vd = h.shape[0], m["heads"], m["dim"], m["vdim"]
    cq, c_new = latents(h, p["dq"], p["dq.norm"], p["dkv"], p["dkv.norm"], eps)
    c = c_new if c_prefix is None else torch.cat([c_prefix, c_new], 0)
    Tk = c.shape[0]
    q = (cq @ p["uq"].T).view(T, H, d)
    k = (c @ p["uk"].T).view(Tk, H, d)
    v = (c @ p["uv"].T).view(Tk, H, vd)
    s = latent_attention_scores(q, k, m["scale"])
    # query i sits at position Tk - T + i and sees every j <= that
    qpos = torch.arange(Tk - T, Tk).view(1, T, 1)
    kpos = torch.arange(Tk).view(1, 1, Tk)
    s = s.masked_fill(kpos > qpos, float("-inf"))
    a = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", a, v).reshape(T, H * vd)
    return o @ p["o"].T, c


def dense_ff(h, gate, up, down):
    return (gelu_tanh(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, correction, top: int, scale: float):
    """(chosen experts [T, top], their weights [T, top]): sigmoid scores, choice biased by `correction`,
    weights from the unbiased scores of the chosen, normalised, times scale."""
    s = torch.sigmoid(h @ router.T)
    idx = torch.topk(s + correction, top, dim=-1).indices
    sel = torch.gather(s, 1, idx)
    return idx, sel / (sel.sum(-1, keepdim=True) + 1e-20) * scale


def expert_ff(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def moe_ff(h, p: Dict[str, torch.Tensor], f: dict):
    r = f["router"]
    idx, wts = route(h, p["router"], p["correction"], r["top"], r["scale"])
    out = torch.zeros(h.shape[0], p["e0.down"].shape[0])
    for t in range(h.shape[0]):
        for j in range(r["top"]):
            e = int(idx[t, j])
            out[t] += wts[t, j] * expert_ff(h[t], p[f"e{e}.up"], p[f"e{e}.down"])
    if f.get("shared"):
        out = out + expert_ff(h, p["shared.up"], p["shared.down"]) * torch.sigmoid(h @ p["shared.sg"].T)
    return out


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer_runs(cfg: dict) -> List[tuple]:
    """(layer, pass, embedding re-added before it) in execution order."""
    n = len(cfg["layers"])
    lp = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    runs = [(i, 0, False) for i in range(lp["start"])]
    for t in range(lp["times"] if lp["stop"] > lp["start"] else 0):
        runs += [(i, t, t > 0 and i == lp["start"]) for i in range(lp["start"], lp["stop"])]
    return runs + [(i, 0, False) for i in range(lp["stop"], n)]


class KaruzenOracle:
    """Whole-model forward over ONE sequence with an explicit latent cache per layer run, so that the
    same object serves whole prompts, portions and token-by-token decoding."""

    def __init__(self, cfg: dict, weights: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.w = {k: v.float() for k, v in weights.items()}
        self.runs = layer_runs(cfg)
        self.eps = cfg["norm"]["eps"]

    def new_cache(self) -> List[Optional[torch.Tensor]]:
        return [None] * len(self.runs)

    def forward(self, tokens: List[int], cache: Optional[list] = None, residuals: Optional[list] = None) -> torch.Tensor:
        """Logits [len(tokens), V] of the new tokens; `cache` (from new_cache) is extended in place."""
        w, cfg = self.w, self.cfg
        cache = cache if cache is not None else self.new_cache()
        x0 = w["embed"][torch.tensor(tokens, dtype=torch.long)]
        x = x0.clone()
        for k, (i, _, readd) in enumerate(self.runs):
            if readd:
                x = x + x0
            ly = cfg["layers"][i]
            h = dyt(x, w[f"l{i}.norm1"], w[f"l{i}.norm1.b"], w[f"l{i}.norm1.alpha"])
            mix, cache[k] = latent_attention(h, sub(w, f"l{i}.mix."), ly["mixer"], self.eps, cache[k])
            f = ly.get("mlp")
            if f is None:
                ff = 0.0
            elif f["kind"] == "dense":
                ff = dense_ff(h, w[f"l{i}.mlp.gate"], w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"])
            else:
                ff = moe_ff(h, sub(w, f"l{i}.mlp."), f)
            x = x + (mix + ff)
            if residuals is not None:
                residuals.append(x.clone())
        return dyt(x, w["final.norm"], w["final.norm.b"], w["final.norm.alpha"]) @ w["embed"].T


def make_config(vocab=320, width=192, layers=None, loop=None, eps=1e-5) -> dict:
    return {"architecture": "Karuzen", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": layers, "loop": loop}


def mixer_cfg(heads=4, dim=32, vdim=48, kv_rank=96, q_rank=40, scale=0.2) -> dict:
    return {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale}


def dense_cfg(ff=160) -> dict:
    return {"kind": "dense", "ff": ff}


def moe_cfg(experts=6, top=2, ff=48, scale=1.5, shared_ff=80) -> dict:
    c = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale}, "expert": {"ff": ff}}
    if shared_ff:
        c["shared"] = {"ff": shared_ff}
    return c


def make_weights(cfg: dict, seed: int = 0, bf16_values: bool = True) -> Dict[str, torch.Tensor]:
    """Random weights under the checkpoint's names.  Values are bf16-representable by default so that the
    bf16 and fp32 paths load identical numbers."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def rnd(*shape, s=1.0):
        t = torch.randn(*shape, generator=g) * s
        return t.bfloat16().float() if bf16_values else t

    def fix(t):
        return t.bfloat16().float() if bf16_values else t

    def norm(prefix):
        return {prefix: fix(1.0 + rnd(W, s=0.2)), prefix + ".b": rnd(W, s=0.1), prefix + ".alpha": fix(0.5 + 0.3 * torch.rand((), generator=g))}

    w = {"embed": rnd(cfg["vocab"], W, s=1.0)}
    w.update(norm("final.norm"))
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        w.update(norm(p + "norm1"))
        H, d, vd, kr, qr = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        w[p + "mix.dq"] = rnd(qr, W, s=W ** -0.5)
        w[p + "mix.dq.norm"] = fix(1.0 + rnd(qr, s=0.2))
        w[p + "mix.uq"] = rnd(H * d, qr, s=qr ** -0.5)
        w[p + "mix.dkv"] = rnd(kr, W, s=W ** -0.5)
        w[p + "mix.dkv.norm"] = fix(1.0 + rnd(kr, s=0.2))
        w[p + "mix.uk"] = rnd(H * d, kr, s=kr ** -0.5)
        w[p + "mix.uv"] = rnd(H * vd, kr, s=kr ** -0.5)
        w[p + "mix.o"] = rnd(W, H * vd, s=(H * vd) ** -0.5)
        f = ly.get("mlp")
        if f is None:
            continue
        if f["kind"] == "dense":
            w[p + "mlp.gate"] = rnd(f["ff"], W, s=W ** -0.5)
            w[p + "mlp.up"] = rnd(f["ff"], W, s=W ** -0.5)
            w[p + "mlp.down"] = rnd(W, f["ff"], s=f["ff"] ** -0.5)
        else:
            E, ef = f["router"]["experts"], f["expert"]["ff"]
            w[p + "mlp.router"] = rnd(E, W, s=2.0 * W ** -0.5)
            w[p + "mlp.correction"] = rnd(E, s=0.3)
            for e in range(E):
                w[p + f"mlp.e{e}.up"] = rnd(ef, W, s=W ** -0.5)
                w[p + f"mlp.e{e}.down"] = rnd(W, ef, s=ef ** -0.5)
            if f.get("shared"):
                sf = f["shared"]["ff"]
                w[p + "mlp.shared.up"] = rnd(sf, W, s=W ** -0.5)
                w[p + "mlp.shared.down"] = rnd(W, sf, s=sf ** -0.5)
                w[p + "mlp.shared.sg"] = rnd(1, W, s=W ** -0.5)
    return w
