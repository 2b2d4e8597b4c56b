"""Repudra (parallel blocks: softmax attention beside an mLSTM matrix memory, gated linear attention, delta rule with a
decay per key channel; one residual with layer scale; xIELU feed-forward) against the plain oracle in
``repudra_oracle.py``.  Every test builds its own small configuration and random checkpoint on disk, so the config
reader, the loader, the page allocator, the batch slots and the chunk path of the runner are all on the tested path.
The GPU tests run the float32 mode at tight tolerance (it shows an off-by-one key, a lost state or a missing tail at
once) and the bf16 serving mode at rounding tolerance.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import pytest
import torch

import repudra_oracle as O

from bee2bee_b200.models.config import ModelConfig, RotarySpec, resolve_config

gpu = pytest.mark.gpu


# ----------------------------------------------------------------------------------------------- model builders
def mlp(ff):
    return {"ff": ff, "kind": "dense"} if ff else None


def par(heads=4, kv=2, dim=16, vdim=24, rot=8, scaling=True, scale=None, rheads=2, rdim=16, rvdim=8, cap=10.0, ff=0):
    left = {"dim": dim, "heads": heads, "kv_heads": kv, "scale": scale if scale is not None else dim ** -0.5, "vdim": vdim}
    if rot:
        left["rot"] = {"base": 5000.0, "dims": rot}
        if scaling:
            left["rot"]["scaling"] = {"factor": 4.0, "fast": 16.0, "original": 64, "slow": 2.0}
    right = {"dim": rdim, "heads": rheads, "vdim": rvdim, "gate_cap": cap}
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp(ff)}


def gla(heads=2, dim=16, vdim=24, tau=8.0, ff=0):
    return {"type": "gla", "mixer": {"dim": dim, "heads": heads, "tau": tau, "vdim": vdim}, "mlp": mlp(ff)}


def cdelta(heads=4, kv=2, dim=16, vdim=8, conv=3, ff=0):
    return {"type": "channel_delta", "mixer": {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv, "vdim": vdim},
            "mlp": mlp(ff)}


def make_cfg(layers, width=64, vocab=200, eps=1e-5, cap=12.0, scale=None):
    return {"architecture": "Repudra", "embedding": {"scale": scale if scale is not None else math.sqrt(width)},
            "layers": layers, "logit_softcap": cap, "norm": {"eps": eps}, "vocab": vocab, "width": width}


def make_tensors(cfg, seed=0, rank=6, tweak=None):
    """random checkpoint (values exactly representable in bf16, kept as float32)"""
    g = torch.Generator().manual_seed(seed)
    W, t = cfg["width"], {}

    def rn(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).bfloat16().float()

    def lin(n_out, n_in, gain=1.0):
        return rn(n_out, n_in, std=gain * n_in ** -0.5)

    t["embed"] = rn(cfg["vocab"], W, std=1.0 / cfg["embedding"]["scale"])
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        t[p + "norm1"] = rn(1, std=0.1, mean=1.0).reshape(())
        if lay["type"] == "parallel":
            a, q = m["left"], p + "mix.left."
            H, G, D, V = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            t[q + "q"], t[q + "k"], t[q + "v"] = lin(H * D, W), lin(G * D, W), lin(G * V, W)
            t[q + "q.norm"], t[q + "k.norm"] = rn(H * D, std=0.1, mean=1.0), rn(G * D, std=0.1, mean=1.0)
            t[q + "o"] = lin(W, H * V)
            r, q = m["right"], p + "mix.right."
            H, D, V = r["heads"], r["dim"], r["vdim"]
            t[q + "q"], t[q + "k"], t[q + "v"], t[q + "g"] = lin(H * D, W), lin(H * D, W), lin(H * V, W), lin(H * V, W)
            t[q + "o"], t[q + "norm"] = lin(W, H * V), rn(H * V, std=0.1, mean=1.0)
            t[q + "i"], t[q + "i.b"] = lin(H, W, 2.0), rn(H, std=0.5)
            t[q + "f"], t[q + "f.b"] = lin(H, W, 2.0), rn(H, std=0.5, mean=2.0)
            t[p + "mix.left.out"], t[p + "mix.right.out"] = rn(W, std=0.1, mean=1.0), rn(W, std=0.1, mean=1.0)
        elif lay["type"] == "gla":
            q = p + "mix."
            H, D, V = m["heads"], m["dim"], m["vdim"]
            t[q + "q"], t[q + "k"], t[q + "v"], t[q + "g"] = lin(H * D, W), lin(H * D, W), lin(H * V, W), lin(H * V, W)
            t[q + "o"], t[q + "norm"] = lin(W, H * V), rn(V, std=0.1, mean=1.0)
            t[q + "a1"], t[q + "a2"], t[q + "a2.b"] = lin(rank, W), lin(H * D, rank, 2.0), rn(H * D, std=1.0, mean=1.0)
        else:
            q = p + "mix."
            H, G, D, V, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            for n, rows in (("q", G * D), ("k", G * D), ("v", H * V)):
                t[q + n], t[q + n + ".conv"] = lin(rows, W, 2.0), rn(rows, taps, std=taps ** -0.5)
            t[q + "b"], t[q + "A_log"], t[q + "norm"] = lin(H, W, 2.0), rn(H, std=0.5, mean=-1.0), rn(V, std=0.1, mean=1.0)
            t[q + "a1"], t[q + "a2"], t[q + "dt_bias"] = lin(rank, W), lin(H * D, rank, 2.0), rn(H * D, std=0.5)
            t[q + "g1"], t[q + "g2"] = lin(rank + 1, W), lin(H * V, rank + 1, 2.0)
            t[q + "o"] = lin(W, H * V)
        if lay["mlp"]:
            f = lay["mlp"]["ff"]
            t[p + "mlp.up"], t[p + "mlp.down"], t[p + "mlp.act"] = lin(f, W), lin(W, f), rn(2, std=0.5)
            t[p + "ls2"] = rn(W, std=0.1, mean=0.6)
        t[p + "ls1"] = rn(W, std=0.1, mean=0.6)
    t["final.norm"] = rn(1, std=0.1, mean=1.0).reshape(())
    t["head"] = lin(cfg["vocab"], W, 3.0)
    if tweak:
        tweak(t)
    return t


def save_model(path, cfg, t):
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.bfloat16().contiguous() for k, v in t.items()}, os.path.join(path, "model.safetensors"))
    return str(path)


def oracle_logits(tokens, t, cfg):
    t64 = {k: v.double() for k, v in t.items()}
    with torch.no_grad():
        return O.forward(torch.tensor(tokens), t64, cfg)[0].float().numpy()


def rel_err(got, want):
    """per-row error: difference with its mean removed (a shift of all logits changes no probability), as a root mean
    square relative to the spread of the logits"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / want.std()


TOL = {torch.float32: 2e-4, torch.bfloat16: 6e-2}


def engine(path, dtype, max_tokens=512, slots=4, chunk_tokens=256):
    from bee2bee_b200.engine.core import Engine

    return Engine(path, device="cuda:0", max_batch=slots, max_seq_len=max_tokens, max_prefill_tokens=chunk_tokens,
                  num_pages=max_tokens // 64 + 1, dtype=dtype, max_logit_rows=chunk_tokens, prefix_cache=False)


def replay(eng, key, tokens, cuts, end=True):
    """feed ``tokens`` in portions ``cuts`` (then single tokens), asking for every position -> [T, V]"""
    out, pos, k = [], 0, 0
    while pos < len(tokens):
        n = min(cuts[k] if k < len(cuts) else 1, len(tokens) - pos)
        k += 1
        last = pos + n == len(tokens)
        out.append(eng.replay_step([(key, tokens[pos:pos + n], list(range(n)))], [key] if (last and end) else []))
        pos += n
    return np.concatenate(out)


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


# ------------------------------------------------------------------------------------------------- CPU tests
def test_config_reader_roundtrip_and_registry():
    d = make_cfg([par(ff=48), gla(ff=0), cdelta(ff=40), par(rot=0, kv=4)])
    c = ModelConfig.from_hf_dict(d, "x")
    assert c.family == "repudra" and c.hybrid and c.recurrent and c.n_layers == 4
    assert c.block_layout == "parallel" and c.scalar_norm and c.layer_scale and c.final_softcap == 12.0
    assert [sp.mixer for sp in c.layer_specs] == ["parallel", "gla", "channel_delta", "parallel"]
    left, right = c.layer_specs[0].sub
    assert (left.mixer, left.heads, left.kv_heads, left.dim, left.vdim) == ("softmax_attention", 4, 2, 16, 24)
    assert left.rot.dims == 8 and left.rot.factor == 4.0 and left.rot.original == 64 and left.rot.slow == 2.0
    assert (right.mixer, right.heads, right.dim, right.vdim, right.gate_cap) == ("mlstm", 2, 16, 8, 10.0)
    assert c.layer_specs[3].sub[0].rot is None and c.layer_specs[1].tau == 8.0 and c.layer_specs[2].conv == 3
    assert c.layer_specs[0].ff == 48 and c.layer_specs[1].ff == 0 and c.embed_scale == 8.0
    assert ModelConfig.from_hf_dict(c.to_hf_dict(), "x") == c
    from bee2bee_b200.models import piece_class
    from bee2bee_b200.models.hybrid import HybridPiece
    assert piece_class(c) is HybridPiece
    with pytest.raises(ValueError):
        ModelConfig.from_hf_dict(make_cfg([{"type": "nope", "mixer": {}, "mlp": None}]), "x")
    with pytest.raises(ValueError):
        ModelConfig.from_hf_dict(make_cfg([par(heads=3, kv=2)]), "x")


def test_rotary_frequency_table_matches_the_oracle():
    for rot in ({"base": 5000.0, "dims": 8}, {"base": 250.0, "dims": 12, "scaling": {"factor": 4.0, "fast": 16.0,
                                                                                    "original": 64, "slow": 2.0}},
                {"base": 1e6, "dims": 32, "scaling": {"factor": 16.0, "fast": 32.0, "original": 4096, "slow": 1.0}}):
        sc = rot.get("scaling") or {}
        spec = RotarySpec(dims=rot["dims"], base=rot["base"], factor=sc.get("factor", 0.0), original=sc.get("original", 0),
                          fast=sc.get("fast", 32.0), slow=sc.get("slow", 1.0))
        pos = torch.tensor([0, 1, 7, 300])
        cos, sin = O.rotary_tables(rot, pos, torch.float64)
        f = torch.tensor(spec.frequencies(), dtype=torch.float64)
        ang = pos.double()[:, None] * f[None, :]
        assert torch.allclose(torch.cos(ang) * spec.amplitude, cos, atol=1e-12)
        assert torch.allclose(torch.sin(ang) * spec.amplitude, sin, atol=1e-12)
        if sc:   # the blend really changes something: the slowest pair is slowed by the full factor
            plain = rot["base"] ** (-2.0 * (rot["dims"] // 2 - 1) / rot["dims"])
            assert abs(f[-1].item() - plain / sc["factor"]) < 1e-12 and abs(f[0].item() - 1.0) < 1e-12


def test_checkpoint_loader_names_and_shapes(tmp_path):
    from bee2bee_b200.models.weights import hybrid_tensor_specs, init_random, load_or_init

    d = make_cfg([par(ff=40), gla(), cdelta()], width=48)
    t = make_tensors(d, rank=5)
    path = save_model(tmp_path / "m", d, t)
    c = resolve_config(path)
    got = load_or_init(path, c, range(3), True, True)
    assert set(got) == set(t)
    for k in t:
        assert torch.equal(got[k], t[k]), k
    assert got["l1.mix.a1"].shape == (5, 48) and got["l2.mix.g1"].shape == (6, 48)   # ranks are the tensors', not the config's
    assert got["l0.norm1"].shape == () and got["final.norm"].shape == ()
    preset = resolve_config("tiny-repudra")
    rnd = init_random(preset, range(preset.n_layers), True, True)
    assert {n for n, _, _ in hybrid_tensor_specs(preset, range(preset.n_layers), True, True)} == set(rnd)


def test_oracle_state_and_cache_carry_over():
    """the oracle's own mechanisms agree with themselves when a sequence is cut (guards the tests below)"""
    d = make_cfg([par(), gla(), cdelta(conv=4)])
    t = {k: v.double() for k, v in make_tensors(d).items()}
    h = torch.randn(11, 64, dtype=torch.float64)
    for i, fn in ((1, O.gla), (2, O.channel_delta)):
        m, p = d["layers"][i]["mixer"], f"l{i}.mix."
        full, _ = fn(h, t, p, m, 1e-5)
        for cut in (1, 2, 9):          # also portions shorter than the convolution
            a, st = fn(h[:cut], t, p, m, 1e-5)
            b, _ = fn(h[cut:], t, p, m, 1e-5, state=st)
            assert torch.allclose(torch.cat([a, b]), full, atol=1e-12)
    m, p = d["layers"][0]["mixer"], "l0.mix."
    full, _ = O.parallel_mixer(h, t, p, m, 1e-5)
    a, st = O.parallel_mixer(h[:7], t, p, m, 1e-5)
    b, _ = O.parallel_mixer(h[7:], t, p, m, 1e-5, pos0=7, state=st)
    assert torch.allclose(torch.cat([a, b]), full, atol=1e-12)


def test_cpu_engine_refuses_hybrid_models():
    from bee2bee_b200.engine.core import Engine

    with pytest.raises(ValueError):
        Engine("tiny-repudra", device="cpu")


# ------------------------------------------------------------------------------------------- kernels alone (GPU)
@gpu
@pytest.mark.parametrize("W", [72, 50, 1040, 1034])       # narrow / wide rows, with and without 16-byte accesses
def test_join_kernel_layer_scale_width_norm_and_scalar_gain(W):
    from bee2bee_b200 import ops

    dev, T, eps = "cuda", 7, 1e-5
    ld = (W + 63) // 64 * 64
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, W, generator=g)
    ys = [torch.randn(T, ld, generator=g) * s for s in (1.0, 3.0, 0.5)]
    ws = [torch.randn(W, generator=g), torch.randn(W, generator=g), None]
    gain = torch.tensor([1.3])
    new = x + O.rms(ys[0][:, :W], eps) * ws[0] + O.rms(ys[1][:, :W], eps) * ws[1] + ys[2][:, :W]
    want_h = O.scalar_norm(new, gain, eps)
    i32 = dict(dtype=torch.int32, device=dev)
    q_start, q_len = torch.tensor([0, 3], **i32), torch.tensor([3, 4], **i32)
    terms = [(ys[0].to(dev), ws[0].to(dev), True), (ys[1].to(dev), ws[1].to(dev), True), (ys[2].to(dev), None, False)]
    xd, h = x.to(dev).contiguous(), torch.zeros(T, ld, device=dev)
    ops.ls_join(xd, q_start, q_len, 2, 4, terms=terms, gamma=gain.to(dev), eps=eps, h=h)
    assert torch.allclose(xd.cpu(), new, atol=1e-5)
    assert torch.allclose(h[:, :W].cpu(), want_h, atol=1e-5) and float(h[:, W:].abs().max()) == 0.0
    # gathered rows, vector gain, bf16 operand: nothing is written back
    xd2, rows = x.to(dev).contiguous(), torch.tensor([5, 0, 6], **i32)
    vec_gain = torch.randn(W, generator=g)
    h2 = torch.zeros(3, ld, device=dev, dtype=torch.bfloat16)
    ops.ls_join(xd2, q_start, q_len, 2, 4, terms=terms[:1], gamma=vec_gain.to(dev), eps=eps, h=h2, rows=rows, n_rows=3)
    assert torch.equal(xd2.cpu(), x)
    want2 = O.rms(x + O.rms(ys[0][:, :W], eps) * ws[0], eps) * vec_gain
    assert torch.allclose(h2[:, :W].float().cpu(), want2[[5, 0, 6]], atol=3e-2, rtol=1e-2)


@gpu
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_short_convolution_kernel_with_tail(taps):
    from bee2bee_b200 import ops

    dev, C, off = "cuda", 70, 5
    g = torch.Generator().manual_seed(taps)
    w = torch.randn(C, taps, generator=g)
    xa, xb = torch.randn(40, C, generator=g), torch.randn(9, C, generator=g)
    zero = torch.zeros(taps - 1, C)
    want_a, _ = O.short_conv(xa, w, zero)
    want_b, _ = O.short_conv(xb, w, zero)
    want_a, want_b = torch.nn.functional.silu(want_a), torch.nn.functional.silu(want_b)
    tail = torch.full((3, max(1, taps - 1), C), 7.0, device=dev)         # stale values of earlier users of the slots
    i32 = dict(dtype=torch.int32, device=dev)
    got_a, got_b, pa, pb = [], [], 0, 0
    # sequence a in slot 2: portions of 1, 2, 20, 17; sequence b in slot 0 joins later: 3, 1, 5
    for na, nb in ((1, 0), (2, 3), (20, 1), (17, 5)):
        rows = [xa[pa:pa + na]] + ([xb[pb:pb + nb]] if nb else [])
        x = torch.zeros(na + nb, off + C + 3)
        x[:, off:off + C] = torch.cat(rows)
        S = 2 if nb else 1
        q_start, q_len = torch.tensor([0, na][:S], **i32), torch.tensor([na, nb][:S], **i32)
        kv_len, slot = torch.tensor([pa + na, pb + nb][:S], **i32), torch.tensor([2, 0][:S], **i32)
        y = torch.zeros(na + nb, C, device=dev)
        ops.short_conv(x.to(dev), off, w.to(dev), tail, y, q_start, q_len, kv_len, slot, S, max(na, nb))
        got_a.append(y[:na].cpu())
        got_b.append(y[na:].cpu())
        pa, pb = pa + na, pb + nb
    assert torch.allclose(torch.cat(got_a), want_a, atol=1e-5) and torch.allclose(torch.cat(got_b), want_b, atol=1e-5)


@gpu
def test_column_activations_xielu_and_soft_cap():
    from bee2bee_b200 import ops

    z = torch.linspace(-6, 6, 97).repeat(3, 1).contiguous()
    act = torch.tensor([0.3, -0.7])
    want = O.xielu(z.double(), act.double()).float()
    ap = float(torch.nn.functional.softplus(act[0]))
    an = float(0.5 + torch.nn.functional.softplus(act[1]))
    out = torch.zeros(3, 97, device="cuda")
    ops.act_cols(z.cuda(), 0, out, 97, ops.COLS_XIELU, 3, p0=ap, p1=an)
    assert torch.allclose(out.cpu(), want, atol=1e-5)
    ops.act_cols(z.cuda() * 10, 0, out, 97, ops.COLS_SOFTCAP, 3, p0=9.0)
    assert torch.allclose(out.cpu(), 9.0 * torch.tanh(z * 10 / 9.0), atol=1e-5)


# --------------------------------------------------------------------------------------------- models (GPU)
SINGLE = {
    "parallel": lambda: make_cfg([par()]),
    # full rotation (dims = head), no frequency scaling, one key head for all query heads, one memory head, wide values
    "parallel_full_rotation_one_kv_head": lambda: make_cfg([par(heads=3, kv=1, dim=8, vdim=40, rot=8, scaling=False,
                                                                rheads=1, rdim=24, rvdim=40)], width=48),
    "parallel_no_rotation": lambda: make_cfg([par(heads=2, kv=2, dim=24, vdim=8, rot=0, rheads=3, rdim=8, rvdim=24)]),
    "gla": lambda: make_cfg([gla()]),
    "gla_one_wide_head": lambda: make_cfg([gla(heads=1, dim=40, vdim=72, tau=1.0)], width=96),
    "channel_delta": lambda: make_cfg([cdelta()]),
    "channel_delta_equal_heads_two_taps": lambda: make_cfg([cdelta(heads=3, kv=3, dim=24, vdim=40, conv=2)], width=80),
    "feed_forward": lambda: make_cfg([gla(heads=1, dim=8, vdim=8, ff=72)], cap=3.0),
    # key widths of 72 .. 128 channels (the recurrences' widest lane layout; 256 in the next one)
    "wide_keys": lambda: make_cfg([par(heads=2, kv=1, dim=72, vdim=16, rot=8, rheads=1, rdim=96, rvdim=16),
                                   cdelta(heads=2, kv=1, dim=128, vdim=16, conv=4), gla(heads=1, dim=72, vdim=24)]),
    "widest_keys": lambda: make_cfg([gla(heads=1, dim=200, vdim=8), par(rheads=1, rdim=256, rvdim=8)]),
    # nothing is a multiple of 4 or 8: scalar paths of the attention kernels in both modes, heads of 10 / 6 / 22
    # channels, a convolution as long as the kernel allows, no logit cap, an embedding scale of 1
    "odd_sizes": lambda: make_cfg([par(heads=3, kv=1, dim=10, vdim=6, rot=6, rheads=3, rdim=10, rvdim=6, ff=30),
                                   cdelta(heads=3, kv=1, dim=10, vdim=22, conv=8), gla(heads=3, dim=18, vdim=10)],
                                  width=50, vocab=131, cap=0.0, scale=1.0),
}


@gpu
@pytest.mark.parametrize("name", sorted(SINGLE))
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_each_mechanism_alone_whole_prompt(tmp_path, name, dtype):
    cfg = SINGLE[name]()
    t = make_tensors(cfg, seed=3)
    eng = engine(save_model(tmp_path / "m", cfg, t), dtype)
    tokens = toks(45, cfg["vocab"], 5)
    got = replay(eng, "a", tokens, [45])
    eng.close()
    assert rel_err(got, oracle_logits(tokens, t, cfg)).max() < TOL[dtype]


def mixed_cfg():
    # sizes that are neither equal to each other nor powers of two: 3 query heads per kv head, value width != key width,
    # rotation on part of a head, two feed-forward widths, a layer without feed-forward, 2 delta heads per q/k head
    return make_cfg([par(heads=6, kv=2, dim=24, vdim=40, rot=12, rheads=3, rdim=24, rvdim=16, ff=72), gla(heads=3, dim=24, vdim=16),
                     cdelta(heads=4, kv=2, dim=16, vdim=24, conv=4, ff=40), par(heads=2, kv=2, dim=8, vdim=16, rot=8, scaling=False)],
                    width=80, vocab=300)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_portions_decode_and_page_borders(tmp_path, dtype):
    """whole prompt == portions of many sizes (down to 2 tokens, shorter than the convolution, across the 64-token page
    border) == token by token, all equal to the oracle at every position"""
    cfg = mixed_cfg()
    t = make_tensors(cfg, seed=11)
    eng = engine(save_model(tmp_path / "m", cfg, t), dtype)
    tokens = toks(150, cfg["vocab"], 6)
    want = oracle_logits(tokens, t, cfg)
    whole = replay(eng, "w", tokens, [150])
    parts = replay(eng, "p", tokens, [2, 5, 7, 49, 2, 3, 61, 1, 2])          # 63 | 64 | 65 straddled, then singles
    single = replay(eng, "s", tokens[:80], [])
    eng.close()
    tol = TOL[dtype]
    assert rel_err(whole, want).max() < tol
    assert rel_err(parts, want).max() < tol
    assert rel_err(single, want[:80]).max() < tol
    cut_noise = 1e-5 if dtype == torch.float32 else tol
    assert rel_err(parts, whole).max() < cut_noise and rel_err(single, whole[:80]).max() < cut_noise


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_mixed_batches_and_reused_slots_and_pages(tmp_path, dtype):
    """unequal requests in one batch (a long portion beside single tokens beside a new request) equal each alone;
    ended requests give slot, state and pages back and the next ones get exactly those"""
    cfg = mixed_cfg()
    t = make_tensors(cfg, seed=14)
    eng = engine(save_model(tmp_path / "m", cfg, t), dtype, max_tokens=320, slots=3)
    V = cfg["vocab"]
    seqs = {k: toks(n, V, 20 + i) for i, (k, n) in enumerate([("a", 100), ("b", 37), ("c", 66), ("d", 90), ("e", 30)])}
    want = {k: oracle_logits(v, t, cfg) for k, v in seqs.items()}
    got = {k: [] for k in seqs}
    at = {k: 0 for k in seqs}

    def step(plan, end=()):
        entries = []
        for k, n in plan:
            entries.append((k, seqs[k][at[k]:at[k] + n], list(range(n))))
        out = eng.replay_step(entries, list(end))
        o = 0
        for k, n in plan:
            got[k].append(out[o:o + n])
            o += n
            at[k] += n

    step([("a", 60), ("b", 2)])
    step([("a", 1), ("b", 30), ("c", 5)])
    step([("a", 3), ("b", 5), ("c", 61)], end=["b", "c"])            # b and c finish: their slots and pages are free again
    used_before = set(eng.alloc.owned(eng._replay["a"][0]))
    step([("a", 36), ("d", 64), ("e", 2)], end=["a"])                 # d and e reuse them (pool: 5 pages, 3 slots)
    step([("d", 1), ("e", 28)], end=["e"])
    step([("d", 25)], end=["d"])
    eng.close()
    assert used_before and not eng._replay
    for k in seqs:
        g = np.concatenate(got[k])
        assert g.shape[0] == len(seqs[k])
        assert rel_err(g, want[k]).max() < TOL[dtype], k


@gpu
@pytest.mark.parametrize("kind", ["attention", "mlstm", "gla", "channel_delta"])
def test_first_token_shows_hundreds_of_tokens_later(tmp_path, kind):
    """weights chosen so that ONE far token matters.  Attention: the last token's query equals the first token's key
    (mirrored embedding row, mirrored key weights), so that key stands out among hundreds.  mLSTM: only the first
    token opens the input gate and nothing is forgotten.  GLA / delta rule: decays of one.  The first token is then
    changed and the last logits must move, in the oracle and in the engine alike, through prompts cut at other places
    and through decoding."""
    V, W = 200, 64
    X, Y, Z = V - 1, V - 2, V - 3                    # first token, last token, replacement of the first (used nowhere else)

    def tweak(t):
        if kind == "mlstm":
            t["l0.mix.right.f.b"].fill_(30.0)         # log forget gate ~ 0: the memory keeps everything
            t["l0.mix.right.f"].zero_()
            e = t["embed"][X]
            t["l0.mix.right.i"][:] = (30.0 / math.sqrt(W)) * e / e.norm()     # W_i h = 30 for token X, a few units else
            t["l0.mix.right.i.b"].fill_(-20.0)
            t["l0.mix.left.o"].zero_()                # ... and the attention beside it says nothing
        elif kind == "attention":
            t["embed"][Y] = t["embed"][X].flip(0)     # the key weights read the width backwards: k(X) = q(Y), v(X) != v(Y)
            t["l0.mix.left.k"][:] = t["l0.mix.left.q"].flip(1)
            t["l0.mix.left.q.norm"].view(2, 32)[:, :4] *= 0.25     # rotated channels: turned by hundreds of radians between
            t["l0.mix.left.k.norm"][:] = t["l0.mix.left.q.norm"]   # the two positions, they must not drown the match
            t["l0.mix.right.o"].zero_()
        elif kind == "gla":
            t["l0.mix.a2.b"].fill_(30.0)              # decay sigmoid(30)^(1/tau) = 1
            t["l0.mix.a2"].zero_()
        else:
            t["l0.mix.A_log"].fill_(-30.0)            # decay exp(-e^-30 softplus) = 1
            t["embed"][:, 0] = -2.0 / math.sqrt(W)    # one coordinate tells token X from all others ...
            t["embed"][X, 0] = 2.0 / math.sqrt(W)
            t["l0.mix.b"].zero_()
            t["l0.mix.b"][:, 0] = 10.0                # ... and only X writes into the state (write strength 1, others ~ 0)
        for k in t:
            t[k] = t[k].bfloat16().float()

    layer = {"attention": par(heads=2, kv=2, dim=32, vdim=16, rot=4, scale=2.0), "mlstm": par(rheads=2, rdim=16, rvdim=16),
             "gla": gla(heads=2, dim=16, vdim=16), "channel_delta": cdelta(heads=2, kv=1, dim=16, vdim=16)}[kind]
    cfg = make_cfg([layer], width=W, vocab=V)
    t = make_tensors(cfg, seed=21, tweak=tweak)
    tokens = [X] + toks(328, V - 3, 8) + [Y]
    other = [Z] + tokens[1:]
    want, want_o = oracle_logits(tokens, t, cfg), oracle_logits(other, t, cfg)
    seen = rel_err(want_o[-1:], want[-1:]).max()
    assert seen > (1e-3 if kind == "gla" else 0.1)                # the far token is visible at the end
    eng = engine(save_model(tmp_path / "m", cfg, t), torch.float32)
    got = replay(eng, "x", tokens, [300, 13, 3, 2])               # prompt, short portions, then decoding
    got_o = replay(eng, "y", other, [1, 2, 61, 1, 63, 200])       # the first token alone, portions that end on page borders
    eng.close()
    assert rel_err(got, want).max() < 2e-4 and rel_err(got_o, want_o).max() < 2e-4
    if kind in ("attention", "mlstm"):                            # bf16 serving mode: tensor-core attention, graphs
        eng = engine(save_model(tmp_path / "m", cfg, t), torch.bfloat16)
        got = replay(eng, "x", tokens, [300, 13, 3, 2])
        got_o = replay(eng, "y", other, [1, 2, 61, 1, 63, 200])
        eng.close()
        assert rel_err(got[-1:], want[-1:]).max() < 6e-2 and rel_err(got_o[-1:], want_o[-1:]).max() < 6e-2


@gpu
def test_matrix_memory_with_strong_forgetting_and_large_gates(tmp_path):
    """gate pre-activations far into the soft cap, forget gates that wipe the memory within a few tokens and input gates
    that then dominate: the running maximum moves by whole units per token, over tiles, portions and decoding"""
    def tweak(t):
        t["l0.mix.right.f.b"].fill_(-6.0)
        t["l0.mix.right.i.b"].fill_(4.0)
        t["l0.mix.right.i"].mul_(6.0)
        t["l0.mix.right.f"].mul_(6.0)
        t["l0.mix.left.o"].zero_()
        for k in t:
            t[k] = t[k].bfloat16().float()

    cfg = make_cfg([par(rheads=3, rdim=24, rvdim=16, cap=7.0)])
    t = make_tensors(cfg, seed=61, tweak=tweak)
    tokens = toks(140, cfg["vocab"], 10)
    want = oracle_logits(tokens, t, cfg)
    eng = engine(save_model(tmp_path / "m", cfg, t), torch.float32)
    whole = replay(eng, "w", tokens, [140])
    parts = replay(eng, "p", tokens, [33, 2, 31, 1, 64])
    eng.close()
    assert rel_err(whole, want).max() < 2e-4 and rel_err(parts, want).max() < 2e-4


@gpu
def test_long_decoding_single_tokens(tmp_path):
    cfg = make_cfg([cdelta(heads=2, kv=2, dim=32, vdim=32, conv=4), par(heads=2, kv=1, dim=32, vdim=32, rot=16, ff=64),
                    gla(heads=2, dim=32, vdim=32)], width=64)
    t = make_tensors(cfg, seed=31)
    tokens = toks(260, cfg["vocab"], 9)
    want = oracle_logits(tokens, t, cfg)
    for dtype in (torch.float32, torch.bfloat16):
        eng = engine(save_model(tmp_path / f"m{dtype}", cfg, t), dtype)
        got = replay(eng, "x", tokens, [20])                       # 240 single-token steps across 4 page borders
        eng.close()
        assert rel_err(got, want).max() < TOL[dtype]


@gpu
def test_greedy_generation_through_the_scheduler(tmp_path):
    """Engine.generate: admission, chunked prefill, CUDA-graph decode bursts, sampler -- greedy tokens equal the
    oracle's argmax continuation; unequal requests share the batch"""
    from bee2bee_b200.engine.core import Engine, SamplingParams

    cfg = mixed_cfg()
    t = make_tensors(cfg, seed=43)
    path = save_model(tmp_path / "m", cfg, t)
    prompts = [toks(70, cfg["vocab"], 1), toks(9, cfg["vocab"], 2), toks(3, cfg["vocab"], 3)]
    n_new = 12
    want = []
    for p in prompts:
        seq = list(p)
        for _ in range(n_new):
            lg = oracle_logits(seq, t, cfg)[-1]
            top2 = np.sort(lg)[-2:]
            assert top2[1] - top2[0] > 1e-3, "test weights give a near tie: pick another seed"
            seq.append(int(lg.argmax()))
        want.append(seq[len(p):])
    eng = Engine(path, device="cuda:0", max_batch=4, max_seq_len=256, max_prefill_tokens=32, decode_burst=5,
                 dtype=torch.float32)
    sp = SamplingParams(max_new_tokens=n_new, temperature=0.0, repetition_penalty=1.0, ignore_eos=True)
    got = eng.generate(prompts, sp)
    again = eng.generate(prompts[::-1], sp)                        # slots and pages are used a second time
    eng.close()
    assert got == want and again == want[::-1]
    eng = Engine(path, device="cuda:0", max_batch=4, max_seq_len=256, max_prefill_tokens=64, decode_burst=4)
    out = eng.generate(prompts, sp)                                # bf16 serving mode: graphs + tcgen05 GEMMs
    eng.close()
    agree = sum(a == b for g, w in zip(out, want) for a, b in zip(g, w))
    assert all(len(o) == n_new for o in out) and agree >= 0.6 * 3 * n_new


@gpu
def test_preset_generates_with_random_weights():
    from bee2bee_b200.engine.core import Engine, SamplingParams

    eng = Engine("tiny-repudra", device="cuda:0", max_batch=4, max_seq_len=256, decode_burst=4)
    outs = eng.generate([[1, 5, 9, 33, 2, 7, 8, 100], [4, 4, 19]], SamplingParams(max_new_tokens=8, ignore_eos=True))
    eng.close()
    assert all(len(o) == 8 for o in outs)


@gpu
def test_trace_run_command_line(tmp_path):
    """bin/trace_run: steps on stdin, `done <step>` lines on stdout, logits files in --out; slots and pages of ended
    sequences serve the next ones (pool of 192 tokens = 3 pages, 2 slots)"""
    import subprocess
    import sys

    cfg = make_cfg([par(heads=2, kv=1, dim=16, vdim=16, ff=32), cdelta(heads=1, kv=1, dim=16, vdim=16), gla(heads=1)])
    t = make_tensors(cfg, seed=51)
    path = save_model(tmp_path / "m", cfg, t)
    a, b, c = toks(70, cfg["vocab"], 1), toks(40, cfg["vocab"], 2), toks(64, cfg["vocab"], 3)
    steps = [
        {"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}], "end": []},
        {"step": 1, "entries": [{"id": "a", "tokens": a[30:], "want": []}, {"id": "b", "tokens": b[:2], "want": [1]}], "end": ["a"]},
        {"step": 2, "entries": [{"id": "b", "tokens": b[2:], "want": [37]}, {"id": "c", "tokens": c, "want": [0, 63]}],
         "end": ["b", "c"]},
    ]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    for dtype, tol in (("float32", 2e-4), ("bfloat16", 6e-2)):
        res = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", path, "--dtype", dtype,
                              "--out", str(out), "--max-tokens", "192", "--slots", "2"],
                             input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
        assert res.returncode == 0, res.stderr[-2000:]
        assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
        wa, wb, wc = (oracle_logits(x, t, cfg) for x in (a, b, c))
        got0 = np.fromfile(out / "0.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        got1 = np.fromfile(out / "1.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        got2 = np.fromfile(out / "2.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        assert rel_err(got0, wa[[0, 29]]).max() < tol and rel_err(got1, wb[[1]]).max() < tol
        assert rel_err(got2, np.concatenate([wb[[39]], wc[[0, 63]]])).max() < tol
