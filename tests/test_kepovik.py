"""Kepovik (hybrid decoder: sigmoid attention in position blocks, generalized delta rule, residual streams, token-pair
embedding) against the plain oracle in ``kepovik_oracle.py``.  Every test builds its own small configuration and random
checkpoint on disk, so the loader, the config reader, the page allocator, the batch slots and the chunk path of the
runner are all on the tested path.  The GPU tests run the float32 mode at tight tolerance (it shows an off-by-one key or a
lost state at once) and the bf16 serving mode at rounding tolerance.
"""
from __future__ import annotations

import json
import os

import numpy as np
import pytest
import torch

import kepovik_oracle as O

from bee2bee_b200.models.config import ModelConfig, resolve_config

gpu = pytest.mark.gpu


# ----------------------------------------------------------------------------------------------- model builders
def att(heads=4, kv=2, dim=16, vdim=24, chunk=8, ff=0, scale=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv, "scale": scale if scale is not None else dim ** -0.5, "vdim": vdim}
    if chunk:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m, "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def delta(heads=2, dim=16, ff=0):
    return {"type": "general_delta", "mixer": {"dim": dim, "heads": heads},
            "mlp": {"ff": ff, "kind": "dense"} if ff else None}


def make_cfg(layers, width=64, vocab=200, streams=3, mult=0.4, pair=(61, 7, 3), eps=1e-5):
    d = {"architecture": "Kepovik", "layers": layers, "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab,
         "width": width}
    if streams:
        d["streams"] = streams
    if pair:
        d["embedding"] = {"bigram": {"buckets": pair[0], "mul_prev": pair[1], "mul_cur": pair[2]}}
    return d


def make_tensors(cfg, seed=0, rank=8, tweak=None):
    """random checkpoint (values exactly representable in bf16, kept as float32)"""
    g = torch.Generator().manual_seed(seed)
    W, t = cfg["width"], {}

    def rn(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).bfloat16().float()

    t["embed"] = rn(cfg["vocab"], W)
    pair = (cfg.get("embedding") or {}).get("bigram")
    if pair:
        t["bigram"] = rn(pair["buckets"] + 1, W)
    ns = cfg.get("streams", 0)
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        t[p + "norm1"] = rn(W, std=0.1)
        if lay["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            t[p + "mix.q"], t[p + "mix.k"] = rn(H * D, W, std=W ** -0.5), rn(G * D, W, std=W ** -0.5)
            t[p + "mix.v"], t[p + "mix.g"] = rn(G * V, W, std=W ** -0.5), rn(H * V, W, std=W ** -0.5)
            t[p + "mix.q.norm"], t[p + "mix.k.norm"] = rn(D, std=0.1, mean=1.0), rn(D, std=0.1, mean=1.0)
            t[p + "mix.pb"] = rn(H, std=0.5, mean=-1.0)
            t[p + "mix.o"] = rn(W, H * V, std=(H * V) ** -0.5)
        else:
            d = m["heads"] * m["dim"]
            for n in ("r", "k", "v", "g", "a"):
                t[p + "mix." + n] = rn(d, W, std=W ** -0.5)
            t[p + "mix.a.b"], t[p + "mix.w0"] = rn(d, std=0.5), rn(d, std=0.5)
            t[p + "mix.w1"], t[p + "mix.w2"] = rn(rank, W, std=W ** -0.5), rn(d, rank, std=rank ** -0.5)
            t[p + "mix.norm"] = rn(d, std=0.1, mean=1.0)
            t[p + "mix.o"] = rn(W, d, std=d ** -0.5)
        if lay["mlp"]:
            f = lay["mlp"]["ff"]
            t[p + "norm2"] = rn(W, std=0.1)
            t[p + "mlp.up"], t[p + "mlp.down"] = rn(f, W, std=W ** -0.5), rn(W, f, std=f ** -0.5)
        for q in (("hc1", "hc2") if lay["mlp"] else ("hc1",)) if ns else ():
            t[f"{p}{q}.in"] = rn(ns, std=0.2, mean=1.0 / ns)
            t[f"{p}{q}.out"] = rn(ns, std=0.2, mean=1.0)
            t[f"{p}{q}.mix"] = (torch.eye(ns) + torch.randn(ns, ns, generator=g) * 0.2).bfloat16().float()
    t["final.norm"] = rn(W, std=0.1)
    t["head"] = rn(cfg["vocab"], W, std=W ** -0.5)
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
        return O.forward(torch.tensor(tokens), t64, cfg).float().numpy()


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
    """feed ``tokens`` in portions ``cuts`` (cycled; then single tokens), asking for every position -> [T, V]"""
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
    d = make_cfg([att(chunk=8, ff=48), delta(ff=0), att(chunk=0, kv=4)], streams=2)
    c = ModelConfig.from_hf_dict(d, "x")
    assert c.family == "kepovik" and c.hybrid and c.recurrent and c.n_layers == 3 and c.streams == 2
    assert [sp.mixer for sp in c.layer_specs] == ["attention", "general_delta", "attention"]
    assert c.layer_specs[0].chunk == 8 and c.layer_specs[2].chunk == 0 and c.layer_specs[0].ff == 48
    assert c.layer_specs[1].ff == 0 and c.pair_buckets == 61
    assert ModelConfig.from_hf_dict(c.to_hf_dict(), "x") == c
    from bee2bee_b200.models import piece_class
    from bee2bee_b200.models.hybrid import HybridPiece
    from bee2bee_b200.models.native import NativePiece
    assert piece_class(c) is HybridPiece and piece_class(resolve_config("tiny-llama")) is NativePiece
    plain = ModelConfig.from_hf_dict(make_cfg([att()], streams=0, pair=None), "p")
    assert plain.streams == 0 and plain.pair_buckets == 0 and not plain.recurrent


def test_checkpoint_loader_names_and_shapes(tmp_path):
    from bee2bee_b200.models.weights import init_random, kepovik_tensor_specs, load_or_init

    d = make_cfg([att(ff=40), delta()], width=48)
    t = make_tensors(d, rank=5)
    path = save_model(tmp_path / "m", d, t)
    c = resolve_config(path)
    got = load_or_init(path, c, range(2), True, True)
    assert set(got) == set(t)
    for k in t:
        assert torch.equal(got[k], t[k]), k
    assert got["l1.mix.w1"].shape == (5, 48)          # the low rank is the tensor's, not the config's
    rnd = init_random(resolve_config("tiny-kepovik"), range(4), True, True)
    assert {n for n, _, _ in kepovik_tensor_specs(resolve_config("tiny-kepovik"), range(4), True, True)} == set(rnd)


def test_cpu_engine_refuses_hybrid_models():
    from bee2bee_b200.engine.core import Engine

    with pytest.raises(ValueError):
        Engine("tiny-kepovik", device="cpu")


def test_oracle_state_and_cache_carry_over():
    """the oracle's own mechanisms agree with themselves when a sequence is cut (guards the tests below)"""
    d = make_cfg([att(chunk=5), delta()])
    t = {k: v.double() for k, v in make_tensors(d).items()}
    h = torch.randn(11, 64, dtype=torch.float64)
    full, S = O.general_delta(h, t, "l1.mix.", d["layers"][1]["mixer"], 1e-5)
    a, S1 = O.general_delta(h[:4], t, "l1.mix.", d["layers"][1]["mixer"], 1e-5)
    b, S2 = O.general_delta(h[4:], t, "l1.mix.", d["layers"][1]["mixer"], 1e-5, state=S1)
    assert torch.allclose(torch.cat([a, b]), full, atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    full, _ = O.sigmoid_attention(h, t, "l0.mix.", d["layers"][0]["mixer"], 1e-5)
    a, kv = O.sigmoid_attention(h[:7], t, "l0.mix.", d["layers"][0]["mixer"], 1e-5)
    b, _ = O.sigmoid_attention(h[7:], t, "l0.mix.", d["layers"][0]["mixer"], 1e-5, pos0=7, past=kv)
    assert torch.allclose(torch.cat([a, b]), full, atol=1e-12)


# ------------------------------------------------------------------------------------------- kernels alone (GPU)
@gpu
def test_pair_embedding_kernel_first_tokens_and_carried_previous():
    from bee2bee_b200 import ops

    dev, V, W, ns, B = "cuda", 50, 40, 3, 23
    g = torch.Generator().manual_seed(1)
    table, pair = torch.randn(V, W, generator=g), torch.randn(B + 1, W, generator=g)
    cfg = {"embedding": {"bigram": {"buckets": B, "mul_prev": 37, "mul_cur": 9}}}
    seq_a, seq_b = toks(9, V, 2), toks(6, V, 3)
    want_a = O.embed(torch.tensor(seq_a), {"embed": table, "bigram": pair}, cfg)
    want_b = O.embed(torch.tensor(seq_b), {"embed": table, "bigram": pair}, cfg)
    # batch: sequence a continues at position 4 (its previous token comes from the state), b starts at 0
    ids = torch.tensor(seq_a[4:] + seq_b, dtype=torch.int32, device=dev)
    pos = torch.tensor(list(range(4, 9)) + list(range(6)), dtype=torch.int32, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    q_start, q_len = torch.tensor([0, 5], **i32), torch.tensor([5, 6], **i32)
    seq_slot = torch.tensor([2, 0], **i32)
    prev = torch.tensor([7, 7, seq_a[3]], **i32)
    streams = torch.zeros(16, ns, W, device=dev)
    for dt in (torch.float32, torch.bfloat16):
        ops.hyb_embed(ids, pos, q_start, q_len, seq_slot, prev, table.to(dev, dt).contiguous(),
                      pair.to(dev, dt).contiguous(), B, 37, 9, streams, 2, 8)
        want = torch.cat([want_a[4:], want_b])
        if dt == torch.bfloat16:
            want = torch.cat([O.embed(torch.tensor(s), {"embed": table.bfloat16().float(),
                                                        "bigram": pair.bfloat16().float()}, cfg) for s in (seq_a, seq_b)])
            want = torch.cat([want[4:9], want[9:]])
        for s in range(ns):
            assert torch.allclose(streams[:11, s].cpu(), want, atol=1e-6), (dt, s)
    ops.hyb_commit_prev(ids, q_start, q_len, seq_slot, prev, 2)
    assert prev.tolist() == [seq_b[-1], 7, seq_a[-1]]


@gpu
@pytest.mark.parametrize("ns", [1, 2, 4])
def test_stream_mixing_kernel(ns):
    from bee2bee_b200 import ops

    dev, T, W, mult, eps = "cuda", 7, 72, 0.45, 1e-5
    g = torch.Generator().manual_seed(ns)
    x = torch.randn(T, ns, W, generator=g)
    y = torch.randn(T, 128, generator=g)
    mix, outw, inw = torch.randn(ns, ns, generator=g), torch.randn(ns, generator=g), torch.randn(ns, generator=g)
    gamma = torch.randn(W, generator=g) * 0.1
    new = torch.einsum("kj,tkw->tjw", mix, x) + mult * outw[None, :, None] * y[:, None, :W]
    u = torch.einsum("k,tkw->tw", inw, new)
    want_h = O.norm_one_plus(u, gamma, eps)
    st = x.to(dev).contiguous()
    h = torch.zeros(T, 128, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    q_start, q_len = torch.tensor([0, 3], **i32), torch.tensor([3, 4], **i32)
    ops.hc_step(st, q_start, q_len, 2, 4, y=y.to(dev), mix=mix.to(dev), outw=outw.to(dev), mult=mult, inw=inw.to(dev),
                gamma=gamma.to(dev), eps=eps, h=h)
    assert torch.allclose(st.cpu(), new, atol=1e-5)
    assert torch.allclose(h[:, :W].cpu(), want_h, atol=1e-5) and float(h[:, W:].abs().max()) == 0.0
    # gathered rows: nothing written back, rows picked by index
    st2 = x.to(dev).contiguous()
    rows = torch.tensor([5, 0, 6], **i32)
    h2 = torch.zeros(3, 128, device=dev, dtype=torch.bfloat16)
    ops.hc_step(st2, q_start, q_len, 2, 4, y=y.to(dev), mix=mix.to(dev), outw=outw.to(dev), mult=mult, inw=inw.to(dev),
                gamma=gamma.to(dev), eps=eps, h=h2, rows=rows, n_rows=3)
    assert torch.equal(st2.cpu(), x)
    assert torch.allclose(h2[:, :W].float().cpu(), want_h[[5, 0, 6]], atol=2e-2, rtol=1e-2)


# --------------------------------------------------------------------------------------------- models (GPU)
SINGLE = {
    "attention": lambda: make_cfg([att(heads=4, kv=2, dim=16, vdim=24, chunk=8)]),
    "attention_full_causal_plain_residual": lambda: make_cfg([att(heads=3, kv=3, dim=24, vdim=8, chunk=0)], streams=0,
                                                             pair=None, mult=1.0),
    "delta": lambda: make_cfg([delta(heads=2, dim=16)]),
    "delta_wide_head": lambda: make_cfg([delta(heads=1, dim=40)], width=96, streams=1),
    "feed_forward": lambda: make_cfg([att(heads=2, kv=1, dim=8, vdim=8, chunk=4, ff=72)], streams=2),
    # nothing is a multiple of 4: scalar column path of the stream kernel, scalar attention kernel in both modes, a delta
    # head of 10 channels, 7 streams (no compile-time instance), blocks of one position (a query sees only itself)
    "odd_sizes": lambda: make_cfg([att(heads=3, kv=1, dim=10, vdim=6, chunk=1, ff=30), delta(heads=3, dim=10),
                                   att(heads=1, kv=1, dim=18, vdim=22, chunk=5)], width=50, vocab=131, streams=7,
                                  pair=(17, 100003, 99991)),
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
    # blocks of 7 positions, two feed-forward widths, a layer without feed-forward, 3 streams
    return make_cfg([att(heads=6, kv=2, dim=24, vdim=40, chunk=7, ff=72), delta(heads=3, dim=24),
                     att(heads=2, kv=2, dim=8, vdim=16, chunk=70), delta(heads=2, dim=16, ff=40)], width=80, vocab=300,
                    streams=3, mult=0.35, pair=(97, 29, 11))


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_portions_decode_and_page_borders(tmp_path, dtype):
    """whole prompt == portions of many sizes (down to 2 tokens, across the 64-token page border and the block edges)
    == token by token, all equal to the oracle at every position"""
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
    t = make_tensors(cfg, seed=12)
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
def test_block_edges_and_far_state_show(tmp_path):
    """weights chosen so that single keys matter: sharp attention weights (large score scale), and a delta rule that
    neither decays nor removes, so the first token is still in the state hundreds of tokens later"""
    def tweak(t):
        t["l1.mix.w0"].fill_(-30.0)        # decay = exp(-e^-0.5 * sigmoid(-30)) = 1: nothing is forgotten
        t["l1.mix.w2"].zero_()
        t["l1.mix.a.b"].fill_(-30.0)       # removal rate 0
        t["l1.mix.a"].zero_()
        t["l0.mix.pb"].fill_(-2.0)

    cfg = make_cfg([att(heads=2, kv=1, dim=16, vdim=16, chunk=16, scale=3.0), delta(heads=2, dim=16)], streams=2,
                   mult=0.5)
    t = make_tensors(cfg, seed=21, tweak=tweak)
    tokens = toks(330, cfg["vocab"], 8)
    other = [(tokens[0] + 1) % cfg["vocab"]] + tokens[1:]
    want, want_o = oracle_logits(tokens, t, cfg), oracle_logits(other, t, cfg)
    assert rel_err(want_o[-1:], want[-1:]).max() > 1e-3          # the far token is visible at the end
    eng = engine(save_model(tmp_path / "m", cfg, t), torch.float32)
    got = replay(eng, "x", tokens, [300, 13, 3, 2])               # prompt edge inside a block, then decoding over block edges
    got_o = replay(eng, "y", other, [17, 15, 1, 31, 33, 200])
    eng.close()
    assert rel_err(got, want).max() < 2e-4 and rel_err(got_o, want_o).max() < 2e-4


@gpu
def test_long_decoding_single_tokens(tmp_path):
    cfg = make_cfg([delta(heads=2, dim=32), att(heads=2, kv=1, dim=32, vdim=32, chunk=50, ff=64)], width=64, streams=4)
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
    oracle's argmax continuation; two unequal requests share the batch"""
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
def test_trace_run_command_line(tmp_path):
    """bin/trace_run: steps on stdin, `done <step>` lines on stdout, logits files in --out; slots and pages of ended
    sequences serve the next ones (pool of 192 tokens = 3 pages, 2 slots)"""
    import subprocess
    import sys

    cfg = make_cfg([att(heads=2, kv=1, dim=16, vdim=16, chunk=6, ff=32), delta(heads=1, dim=16)], streams=2)
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
