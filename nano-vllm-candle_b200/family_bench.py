"""Karuzen beside the closest existing family (Qwen3, dense GQA) at equal layer sizes: prefill and decode throughput
through LLMEngine, plus per-op times and roofline fractions.  Random weights, synthetic prompts.  Used by
`bench.py --compare-families`; the default benchmark does not touch this module.

Roofline of an op: time_min = max(flops / bf16 peak, bytes / HBM peak) from its algorithmic work (logical sizes, weights
and cache rows once); frac = time_min / measured time."""
from __future__ import annotations

import time
from typing import Dict, List

import numpy as np

BLOCK = 64

# (name, width, heads, ff, layers, moe) - layer shapes of small / mid dense models; head size 128 in both families
SIZES = [
    {"name": "w1024-h16-ff3072", "width": 1024, "heads": 16, "ff": 3072, "layers": 4, "vocab": 32768},
    {"name": "w2048-h16-ff6144", "width": 2048, "heads": 16, "ff": 6144, "layers": 4, "vocab": 32768},
    {"name": "w1024-h16-moe16x2-ff1536", "width": 1024, "heads": 16, "ff": 4608, "layers": 4, "vocab": 32768,
     "moe": {"experts": 16, "top": 2, "expert_ff": 1536, "shared_ff": 1536}},
]
KV_RANK, Q_RANK, DIM = 128, 512, 128


def karuzen_config(sz: dict) -> dict:
    mixer = {"heads": sz["heads"], "dim": DIM, "vdim": DIM, "kv_rank": KV_RANK, "q_rank": Q_RANK, "scale": DIM ** -0.5}
    if "moe" in sz:
        m = sz["moe"]
        mlp = {"kind": "moe", "router": {"experts": m["experts"], "top": m["top"], "scale": 1.0}, "expert": {"ff": m["expert_ff"]},
               "shared": {"ff": m["shared_ff"]}}
    else:
        mlp = {"kind": "dense", "ff": sz["ff"]}
    return {"architecture": "Karuzen", "vocab": sz["vocab"], "width": sz["width"], "norm": {"eps": 1e-5},
            "layers": [{"type": "latent_attention", "mixer": dict(mixer), "mlp": dict(mlp)} for _ in range(sz["layers"])], "loop": None}


def karuzen_weights(cfg: dict, seed: int = 0):
    """(name, bf16 CPU tensor) pairs, generated one at a time."""
    import torch
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i):
        return (torch.randn(o, i, generator=g) * i ** -0.5).bfloat16()

    def norm(p):
        yield p, torch.ones(W).bfloat16()
        yield p + ".b", torch.zeros(W).bfloat16()
        yield p + ".alpha", torch.tensor(0.5).bfloat16()

    yield "embed", (torch.randn(cfg["vocab"], W, generator=g) * 0.05).bfloat16()
    yield from norm("final.norm")
    for i, ly in enumerate(cfg["layers"]):
        m, p = ly["mixer"], f"l{i}."
        yield from norm(p + "norm1")
        H, d, vd, kr, qr = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
        yield p + "mix.dq", mat(qr, W)
        yield p + "mix.dq.norm", torch.ones(qr).bfloat16()
        yield p + "mix.uq", mat(H * d, qr)
        yield p + "mix.dkv", mat(kr, W)
        yield p + "mix.dkv.norm", torch.ones(kr).bfloat16()
        yield p + "mix.uk", mat(H * d, kr)
        yield p + "mix.uv", mat(H * vd, kr)
        yield p + "mix.o", mat(W, H * vd)
        f = ly["mlp"]
        if f["kind"] == "dense":
            yield p + "mlp.gate", mat(f["ff"], W)
            yield p + "mlp.up", mat(f["ff"], W)
            yield p + "mlp.down", mat(W, f["ff"])
        else:
            E, ef, sf = f["router"]["experts"], f["expert"]["ff"], f["shared"]["ff"]
            yield p + "mlp.router", mat(E, W)
            yield p + "mlp.correction", torch.zeros(E).bfloat16()
            for e in range(E):
                yield p + f"mlp.e{e}.up", mat(ef, W)
                yield p + f"mlp.e{e}.down", mat(W, ef)
            yield p + "mlp.shared.up", mat(sf, W)
            yield p + "mlp.shared.down", mat(W, sf)
            yield p + "mlp.shared.sg", mat(1, W)


def _prompts(n, length, vocab, seed):
    rng = np.random.default_rng(seed)
    return [rng.integers(0, vocab, length).tolist() for _ in range(n)]


def _run_engine(eng, runner, vocab, eos, batch_p, batch_d, plen, K, W):
    """(prefill tok/s, decode tok/s, ms per decode step, kernels per decode step) through LLMEngine."""
    nblocks = runner.num_kvcache_blocks
    T = runner.max_num_batched_tokens
    engine = eng.LLMEngine(eng.Scheduler(eng.SchedulerConfig(max(batch_p, batch_d), T, eos, nblocks, BLOCK)), runner, greedy=True)
    best = None
    for rep in range(4):                       # first repetition is the warm-up
        for p in _prompts(batch_p, plen, vocab, 10 + rep):
            engine.add_request(p, eng.SamplingParams(1.0, 1, True))
        t0 = time.perf_counter()
        s = engine.step()                      # synchronous: returns after the tokens are on the host
        dt = time.perf_counter() - t0
        assert s.is_prefill and engine.is_finished()
        if rep > 0:
            best = dt if best is None else min(best, dt)
    for p in _prompts(batch_d, plen, vocab, 3):
        engine.add_request(p, eng.SamplingParams(1.0, W + K + 8, True))
    while engine.num_waiting():
        engine.step()
    for _ in range(max(W, 3)):
        engine.step()
    ms_step, launches = runner.time_decode(K)
    return engine, batch_p * plen / best, batch_d / (ms_step * 1e-3), ms_step, launches


def _roof(flops, nbytes, us, pk):
    tmin = max(flops / (pk["bf16"] * 1e12), nbytes / (pk["hbm"] * 1e9)) * 1e6
    return {"us": round(us, 2), "tflops": round(flops / us / 1e6, 1), "gbs": round(nbytes / us / 1e3, 1), "roofline_frac": round(tmin / us, 3)}


def karuzen_rooflines(cfg, prof: Dict[str, float], N: int, B: int, ctx_lens: List[int], q_lens: List[int], pk) -> dict:
    """Per-op roofline of one profiled step (times summed over the layers; work summed the same way)."""
    L = len(cfg["layers"])
    m, f, W = cfg["layers"][0]["mixer"], cfg["layers"][0]["mlp"], cfg["width"]
    H, d, vd, kr, qr = m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    out = {}

    def gemm(name, o, i, rows=N, copies=1):
        if name in prof:
            out[name] = _roof(L * 2.0 * rows * o * i * copies, L * 2.0 * (o * i * copies + rows * (o + i) * copies), prof[name], pk)

    gemm("gemm_down_latents", qr + kr, W)
    gemm("gemm_uq", H * d, qr)
    gemm("absorb_uk", kr, d, copies=H)
    gemm("absorb_uv", vd, kr, copies=H)
    gemm("gemm_o", W, H * vd)
    if "latent_attn" in prof:
        pairs = sum(q * c - q * (q - 1) // 2 for q, c in zip(q_lens, ctx_lens))       # visible (query, key) pairs
        out["latent_attn"] = _roof(L * 4.0 * H * kr * pairs, L * 2.0 * (sum(ctx_lens) * kr + 2 * N * H * kr), prof["latent_attn"], pk)
    if f["kind"] == "dense":
        gemm("gemm_gate_up", 2 * f["ff"], W)
        gemm("gemm_ff_down", W, f["ff"])
    else:
        E, top, ef, sf = f["router"]["experts"], f["router"]["top"], f["expert"]["ff"], f["shared"]["ff"]
        touched = min(E, N * top)
        for name in ("moe_up", "moe_down"):
            if name in prof:
                out[name] = _roof(L * 2.0 * N * top * ef * W, L * 2.0 * (touched * ef * W + N * top * (ef + W)), prof[name], pk)
        if "shared_expert" in prof:
            out["shared_expert"] = _roof(L * 4.0 * N * sf * W, L * 2.0 * (2 * sf * W + N * (2 * sf + 2 * W)), prof["shared_expert"], pk)
    for name in ("dyt_norm", "latent_norm_store", "gelu_mul", "moe_route", "moe_sort", "moe_gather", "moe_combine", "embed", "final_norm", "lm_head"):
        if name in prof:
            out[name] = {"us": round(prof[name], 2)}
    return out


def compare(ctx_ours, sizes=None, batch_p=16, batch_d=64, plen=512, K=32, W=4, peaks=None) -> dict:
    import importlib
    import torch
    eng = importlib.import_module("nano-vllm-candle_b200.engine")
    synth = importlib.import_module("nano-vllm-candle_b200.synth")
    pk = peaks or {"bf16": 1590.0, "hbm": 6650.0, "source": "fallback"}
    T = batch_p * plen
    nblocks = max(batch_p, batch_d) * (-(-(plen + W + K + 24) // BLOCK)) + 8
    results = []
    for sz in sizes or SIZES:
        rec = {"size": sz["name"]}
        # ---- Karuzen
        cfg = karuzen_config(sz)
        t0 = time.perf_counter()
        kr = eng.ModelRunner.from_config(ctx_ours, cfg, karuzen_weights(cfg), num_kvcache_blocks=nblocks, kvcache_block_size=BLOCK,
                                         max_num_seqs=max(batch_p, batch_d), max_num_batched_tokens=T,
                                         max_model_len=(-(-(plen + W + K + 24) // BLOCK)) * BLOCK)
        load_s = time.perf_counter() - t0
        engine, p_tps, d_tps, ms_step, launches = _run_engine(eng, kr, sz["vocab"], -1, batch_p, batch_d, plen, K, W)
        kr.arm_profile()
        engine.step()                                              # one more decode step, un-captured, with events
        prof_d = kr.profile()
        ctx_d = plen + max(W, 3) + 2
        roof_d = karuzen_rooflines(cfg, prof_d, batch_d, batch_d, [ctx_d] * batch_d, [1] * batch_d, pk)
        engine.close()
        e2 = eng.LLMEngine(eng.Scheduler(eng.SchedulerConfig(batch_p, T, -1, nblocks, BLOCK)), kr, greedy=True)
        for p in _prompts(batch_p, plen, sz["vocab"], 77):
            e2.add_request(p, eng.SamplingParams(1.0, 1, True))
        kr.arm_profile()
        e2.step()
        prof_p = kr.profile()
        roof_p = karuzen_rooflines(cfg, prof_p, T, batch_p, [plen] * batch_p, [plen] * batch_p, pk)
        e2.close()
        rec["karuzen"] = {"prefill_tok_s": round(p_tps), "decode_tok_s": round(d_tps), "decode_ms_per_step": round(ms_step, 4),
                          "kernels_per_decode_step": launches, "weights_load_s": round(load_s, 1),
                          "weight_bytes": kr.weight_bytes(), "cache_bytes_per_token": kr.kv_bytes_per_token(),
                          "prefill_ops": roof_p, "decode_ops": roof_d}
        kr.close()
        torch.cuda.empty_cache()
        # ---- Qwen3 at the same width / heads / ff / layers / vocab (8 kv heads of 128)
        qc = eng.Qwen3Config(vocab_size=sz["vocab"], hidden_size=sz["width"], head_dim=128, num_hidden_layers=sz["layers"],
                             num_attention_heads=sz["heads"], num_key_value_heads=8, intermediate_size=sz["ff"],
                             max_position_embeddings=4096, bos_token_id=1, eos_token_id=2)
        qr_ = eng.Qwen3ModelRunner.from_weights(ctx_ours, qc, synth.iter_weights_device(qc, 0, device="cuda:0"), num_kvcache_blocks=nblocks,
                                                kvcache_block_size=BLOCK, max_num_seqs=max(batch_p, batch_d), max_num_batched_tokens=T,
                                                max_model_len=(-(-(plen + W + K + 24) // BLOCK)) * BLOCK)
        engine, p_tps, d_tps, ms_step, launches = _run_engine(eng, qr_, sz["vocab"], 2, batch_p, batch_d, plen, K, W)
        ops = {op: qr_.time_op(op, 5)[0] * 1e3 for op in ("paged_decode", "gemm_qkv", "gemm_o", "gemm_gate_up", "gemm_down", "rmsnorm",
                                                           "qk_norm_rope")}
        Hh, I, nh = sz["width"], sz["ff"], sz["heads"]
        ctx_d = plen + max(W, 3) + 1 + K
        qroof = {
            "paged_decode": _roof(4.0 * nh * 128 * ctx_d * batch_d, 2.0 * (batch_d * ctx_d * 2 * 8 * 128 + 2 * batch_d * nh * 128), ops["paged_decode"], pk),
            "gemm_qkv": _roof(2.0 * batch_d * Hh * (nh + 16) * 128, 2.0 * Hh * (nh + 16) * 128, ops["gemm_qkv"], pk),
            "gemm_o": _roof(2.0 * batch_d * Hh * nh * 128, 2.0 * Hh * nh * 128, ops["gemm_o"], pk),
            "gemm_gate_up": _roof(4.0 * batch_d * Hh * I, 4.0 * Hh * I, ops["gemm_gate_up"], pk),
            "gemm_down": _roof(2.0 * batch_d * Hh * I, 2.0 * Hh * I, ops["gemm_down"], pk),
            "rmsnorm": {"us": round(ops["rmsnorm"], 2)}, "qk_norm_rope": {"us": round(ops["qk_norm_rope"], 2)},
        }
        rec["qwen3"] = {"prefill_tok_s": round(p_tps), "decode_tok_s": round(d_tps), "decode_ms_per_step": round(ms_step, 4),
                        "kernels_per_decode_step": launches, "weight_bytes": qr_.weight_bytes(),
                        "cache_bytes_per_token": qr_.kv_bytes_per_token(), "decode_ops_per_layer_call": qroof}
        engine.close()
        qr_.close()
        torch.cuda.empty_cache()
        results.append(rec)
    return {"metric": "karuzen_vs_qwen3_equal_layer_sizes", "unit": "tok/s", "dtype": "bf16", "data": "synthetic",
            "workload": {"prefill": f"{batch_p} x {plen} tokens in one step", "decode": f"batch {batch_d} at context ~{plen + W + K}",
                         "timing": "prefill: host wall clock around the synchronous engine step, best of 3 after a warm-up; decode: CUDA events "
                                   "around K replays of the captured step; per-op: CUDA events inside one un-captured step"},
            "peaks": pk, "results": results}
