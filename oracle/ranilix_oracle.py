"""Plain fp32 restatement of the Ranilix design, one function per mechanism, slow on purpose.

Notation: W (width), V (vocab), T (new tokens of one sequence), P (tokens before them).  Linear weights
are [out, in] and act as y = W x.  A layer has two RMS norms of the same x and is parallel:
x <- x + (mixer(n1(x)) + ff(n2(x))).  Two kinds of mixer:

  attention   grouped-query attention with biases on q / k / v, a per-head RMS norm of q and k (one
              weight vector shared by the heads), interleaved rotary pairs (2i, 2i+1) on the first
              rot.dims numbers of a head, a sliding window (query at position i sees i - size < j <= i),
              a softmax whose denominator holds one more term exp(sink_h), values blended with the
              values of the first blending layer, and a sigmoid gate of the layer input on the heads'
              outputs;
  parallel    two mixers on the same input: plain causal grouped-query attention (interleaved rotary,
              no biases / norms / gate) and retention (rotate-half rotary, keys scaled by dim^-1/2, a
              per-head state S <- decay S + k v^T read as S^T q, each head's output divided by its root
              mean square, a silu gate); result = left_scale * left + right_scale * right.

The caches are explicit: every function takes what earlier tokens left and returns what it leaves, so
that the same code serves whole prompts, portions and token-by-token decoding.  Everything here is
float32 torch on the CPU; nothing is shared with the CUDA path.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch


def rms_norm(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def rotary_angles(pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """[T, dims / 2] angles p * base^(-2i / dims)."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    return (pos.double().view(-1, 1) * f.view(1, -1))


def rotary_interleaved(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [T, heads, d]; pairs (2i, 2i + 1) of the first `dims` numbers of every head are turned by the angle."""
    if dims == 0:
        return x
    a = rotary_angles(pos, dims, base)
    c, s = a.cos().float().unsqueeze(1), a.sin().float().unsqueeze(1)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def rotary_half(x: torch.Tensor, pos: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x: [T, heads, d]; number i is paired with number i + dims / 2."""
    if dims == 0:
        return x
    a = rotary_angles(pos, dims, base)
    c, s = a.cos().float().unsqueeze(1), a.sin().float().unsqueeze(1)
    h = dims // 2
    u, v = x[..., :h], x[..., h:dims]
    out = x.clone()
    out[..., :h] = u * c - v * s
    out[..., h:dims] = v * c + u * s
    return out


def softmax_attention(q, k, v, scale: float, qpos: torch.Tensor, window: Optional[int] = None,
                      sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: [T, H, d] at positions qpos; k: [Tk, G, d], v: [Tk, G, vd] at positions 0 .. Tk - 1.  Query head h reads
    key / value head h // (H / G).  Visible: j <= i, and i - j < window when a window is given.  With a sink the
    denominator has one more term exp(sink_h), which carries no value.  Returns [T, H * vd]."""
    T, H, _ = q.shape
    Tk, G, vd = v.shape
    out = torch.zeros(T, H, vd)
    kpos = torch.arange(Tk)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h, :] @ k[:, g, :].T) * scale                      # [T, Tk]
        vis = kpos.view(1, -1) <= qpos.view(-1, 1)
        if window is not None:
            vis &= (qpos.view(-1, 1) - kpos.view(1, -1)) < window
        s = s.masked_fill(~vis, float("-inf"))
        m = s.max(-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].view(1, 1))
        e = torch.exp(s - m)
        den = e.sum(-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h, :] = (e / den) @ v[:, g, :]
    return out.reshape(T, H * vd)


def windowed_attention(h, p: Dict[str, torch.Tensor], m: dict, eps: float, pos0: int, kv_prefix=None,
                       v_first: Optional[torch.Tensor] = None):
    """The 'attention' mixer over T new tokens at positions pos0 ...  kv_prefix = (k, v) of earlier tokens.
    v_first: this step's values of the first blending layer (None in that layer and in layers that do not blend).
    Returns (output [T, W], (k, v) of all tokens, this layer's own unblended values [T, G, vd])."""
    T, H, G, d, vd = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    q = (h @ p["q"].T + p["q.b"]).view(T, H, d)
    k = (h @ p["k"].T + p["k.b"]).view(T, G, d)
    v = (h @ p["v"].T + p["v.b"]).view(T, G, vd)
    q = rms_norm(q, p["q.norm"], eps)
    k = rms_norm(k, p["k.norm"], eps)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotary_interleaved(q, pos, rot["dims"], rot["base"])
    k = rotary_interleaved(k, pos, rot["dims"], rot["base"])
    v_own = v
    if v_first is not None:
        lam = p["vmix"]
        v = (1.0 - lam) * v + lam * v_first.reshape(T, G, vd)      # head by head when the shapes agree, else as one flat row
    if kv_prefix is not None:
        k = torch.cat([kv_prefix[0], k], 0)
        v = torch.cat([kv_prefix[1], v], 0)
    window = (m.get("mask") or {}).get("size")
    o = softmax_attention(q, k, v, m["scale"], pos, window, p["sink"])
    o = o * torch.sigmoid(h @ p["g"].T)
    return o @ p["o"].T, (k, v), v_own


def causal_attention(h, p: Dict[str, torch.Tensor], m: dict, pos0: int, kv_prefix=None):
    """The left half of the 'parallel' mixer: grouped-query causal attention, interleaved rotary, nothing else."""
    T, H, G, d, vd = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotary_interleaved((h @ p["q"].T).view(T, H, d), pos, rot["dims"], rot["base"])
    k = rotary_interleaved((h @ p["k"].T).view(T, G, d), pos, rot["dims"], rot["base"])
    v = (h @ p["v"].T).view(T, G, vd)
    if kv_prefix is not None:
        k = torch.cat([kv_prefix[0], k], 0)
        v = torch.cat([kv_prefix[1], v], 0)
    o = softmax_attention(q, k, v, m["scale"], pos)
    return o @ p["o"].T, (k, v)


def retention(h, p: Dict[str, torch.Tensor], m: dict, eps: float, pos0: int, state: Optional[torch.Tensor] = None):
    """The right half: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t, token by token.  state: [heads, d, vd]
    (None = zeros).  Returns (output [T, W], state after the last token)."""
    T, H, d, vd = h.shape[0], m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(pos0, pos0 + T)
    rot = m.get("rot") or {"dims": 0, "base": 1.0}
    q = rotary_half((h @ p["q"].T).view(T, H, d), pos, rot["dims"], rot["base"])
    k = rotary_half((h @ p["k"].T).view(T, H, d), pos, rot["dims"], rot["base"]) * d ** -0.5
    v = (h @ p["v"].T).view(T, H, vd)
    S = torch.zeros(H, d, vd) if state is None else state.clone()
    decay = torch.tensor(m["decay"], dtype=torch.float32).view(H, 1, 1)
    o = torch.zeros(T, H, vd)
    for t in range(T):
        S = decay * S + k[t].unsqueeze(-1) * v[t].unsqueeze(-2)
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, None, eps).reshape(T, H * vd)
    g = h @ p["g"].T
    o = o * (g * torch.sigmoid(g))
    return o @ p["o"].T, S


def dense_ff(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


class RanilixOracle:
    """Whole-model forward over ONE sequence with an explicit cache, so that the same object serves whole prompts,
    portions and token-by-token decoding.  cache = {"len": tokens so far, "layers": [per-layer dict]}."""

    def __init__(self, cfg: dict, weights: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.w = {k: v.float() for k, v in weights.items()}
        self.eps = cfg["norm"]["eps"]
        blend = [i for i, ly in enumerate(cfg["layers"]) if ly["type"] == "attention" and ly["mixer"].get("v_mix")]
        self.first_blend = blend[0] if blend else -1

    def new_cache(self) -> dict:
        return {"len": 0, "layers": [dict() for _ in self.cfg["layers"]]}

    def forward(self, tokens: List[int], cache: Optional[dict] = None, residuals: Optional[list] = None) -> torch.Tensor:
        """Logits [len(tokens), V] of the new tokens; `cache` (from new_cache) is extended in place."""
        w, cfg = self.w, self.cfg
        cache = cache if cache is not None else self.new_cache()
        pos0 = cache["len"]
        x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
        v_first = None
        for i, ly in enumerate(cfg["layers"]):
            c = cache["layers"][i]
            m = ly["mixer"]
            h1 = rms_norm(x, w[f"l{i}.norm1"], self.eps)
            h2 = rms_norm(x, w[f"l{i}.norm2"], self.eps)
            if ly["type"] == "attention":
                blends = bool(m.get("v_mix"))
                mix, c["kv"], v_own = windowed_attention(h1, sub(w, f"l{i}.mix."), m, self.eps, pos0, c.get("kv"),
                                                         v_first if blends and i != self.first_blend else None)
                if i == self.first_blend:
                    v_first = v_own
            elif ly["type"] == "parallel":
                left, c["kv"] = causal_attention(h1, sub(w, f"l{i}.mix.left."), m["left"], pos0, c.get("kv"))
                right, c["state"] = retention(h1, sub(w, f"l{i}.mix.right."), m["right"], self.eps, pos0, c.get("state"))
                mix = m["left_scale"] * left + m["right_scale"] * right
            else:
                raise ValueError(ly["type"])
            f = ly.get("mlp")
            ff = dense_ff(h2, w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"]) if f is not None else 0.0
            x = x + (mix + ff)
            if residuals is not None:
                residuals.append(x.clone())
        cache["len"] = pos0 + len(tokens)
        return rms_norm(x, w["final.norm"], self.eps) @ w["head"].T


# ------------------------------------------------------------------------------------------ small configurations

def attention_cfg(heads=4, kv_heads=2, dim=32, vdim=24, window=12, rot_dims=16, rot_base=10000.0, scale=0.2, v_mix=True) -> dict:
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "v_mix": v_mix,
         "rot": {"dims": rot_dims, "base": rot_base}}
    if window is not None:
        m["mask"] = {"size": window}
    return {"type": "attention", "mixer": m}


def parallel_cfg(heads=4, kv_heads=2, dim=32, vdim=40, rot_dims=8, rot_base=10000.0, scale=0.18, left_scale=1.1,
                 r_heads=3, r_dim=16, r_vdim=24, r_rot_dims=16, r_rot_base=5000.0, decay=(0.9, 0.97, 0.995), right_scale=0.6) -> dict:
    return {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot_dims, "base": rot_base}},
        "left_scale": left_scale,
        "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay), "rot": {"dims": r_rot_dims, "base": r_rot_base}},
        "right_scale": right_scale}}


def with_mlp(layer: dict, ff: Optional[int] = 96) -> dict:
    layer = dict(layer)
    layer["mlp"] = {"kind": "dense", "ff": ff} if ff else None
    return layer


def make_config(vocab=200, width=96, layers=None, eps=1e-5, embedding_scale=3.0) -> dict:
    return {"architecture": "Ranilix", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "embedding": {"scale": embedding_scale}, "layers": layers}


def make_weights(cfg: dict, seed: int = 0, bf16_values: bool = True) -> Dict[str, torch.Tensor]:
    """Random weights under the checkpoint's names; values bf16-representable by default so that the bf16 and fp32
    paths load identical numbers."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def fix(t):
        return t.bfloat16().float() if bf16_values else t

    def rnd(*shape, s=1.0):
        return fix(torch.randn(*shape, generator=g) * s)

    w = {"embed": rnd(cfg["vocab"], W, s=1.0 / cfg["embedding"]["scale"]), "final.norm": fix(1.0 + rnd(W, s=0.2)),
         "head": rnd(cfg["vocab"], W, s=W ** -0.5)}
    for i, ly in enumerate(cfg["layers"]):
        p, m = f"l{i}.", ly["mixer"]
        w[p + "norm1"] = fix(1.0 + rnd(W, s=0.2))
        w[p + "norm2"] = fix(1.0 + rnd(W, s=0.2))
        if ly["type"] == "attention":
            H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            for n, rows in (("q", H * d), ("k", G * d), ("v", G * vd)):
                w[p + "mix." + n] = rnd(rows, W, s=W ** -0.5)
                w[p + "mix." + n + ".b"] = rnd(rows, s=0.2)
            w[p + "mix.q.norm"] = fix(1.0 + rnd(d, s=0.3))
            w[p + "mix.k.norm"] = fix(1.0 + rnd(d, s=0.3))
            w[p + "mix.vmix"] = fix(0.2 + 0.5 * torch.rand((), generator=g))
            w[p + "mix.sink"] = rnd(H, s=1.0)
            w[p + "mix.g"] = rnd(H * vd, W, s=W ** -0.5)
            w[p + "mix.o"] = rnd(W, H * vd, s=(H * vd) ** -0.5)
        else:
            L, R = m["left"], m["right"]
            H, G, d, vd = L["heads"], L["kv_heads"], L["dim"], L["vdim"]
            w[p + "mix.left.q"] = rnd(H * d, W, s=W ** -0.5)
            w[p + "mix.left.k"] = rnd(G * d, W, s=W ** -0.5)
            w[p + "mix.left.v"] = rnd(G * vd, W, s=W ** -0.5)
            w[p + "mix.left.o"] = rnd(W, H * vd, s=(H * vd) ** -0.5)
            H, d, vd = R["heads"], R["dim"], R["vdim"]
            w[p + "mix.right.q"] = rnd(H * d, W, s=W ** -0.5)
            w[p + "mix.right.k"] = rnd(H * d, W, s=W ** -0.5)
            w[p + "mix.right.v"] = rnd(H * vd, W, s=W ** -0.5)
            w[p + "mix.right.g"] = rnd(H * vd, W, s=W ** -0.5)
            w[p + "mix.right.o"] = rnd(W, H * vd, s=(H * vd) ** -0.5)
        f = ly.get("mlp")
        if f is not None:
            w[p + "mlp.up"] = rnd(f["ff"], W, s=W ** -0.5)
            w[p + "mlp.down"] = rnd(W, f["ff"], s=f["ff"] ** -0.5)
    return w
