"""A piece of a *hybrid* decoder (family ``kepovik``) on one B200: layers whose token mixer is either gated sigmoid
attention over the paged KV cache or a generalized delta-rule recurrence with a per-sequence fp32 state, joined by
several residual streams (hyper-connections), behind a token + hashed token-pair embedding.

Same interface as ``native.NativePiece`` (the runner drives both through ``forward(BatchMeta)``): a flat batch of spans
(prompt portions of any length beside single decoded tokens), physical KV slots and block tables from the page allocator,
logits for the rows named by ``last_idx``.  What is new here and lives next to the shared machinery:

* ``state`` / ``prev_tok``: one recurrent state per delta-rule layer and the last token, indexed by the *batch slot*
  of the sequence (``BatchMeta.seq_slot``); a span that starts at position 0 starts from a zero state, so a slot that is
  used again needs no clearing.
* ``streams``: the residual is ``[tokens, streams, width]`` in fp32; ``ops.hc_step`` applies the stream mixing of the
  sublayer that just ran and produces the normed input of the next one in a single pass.
* precision: streams, norms, scores, decays and the state are fp32 in every mode; ``dtype`` only selects what feeds the
  matrix products and what the KV cache holds (bf16 on the tcgen05 GEMM, or float32 through cuBLAS for bit-faithful runs).

Launches per layer: attention 5 (+3 with a feed-forward), delta rule 7.  The reference has no counterpart
(it delegates every architecture to ``transformers``, /root/reference/bee2bee/hf.py:23-44).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Iterable, Optional

import torch

from .. import ops
from .config import LayerSpec, ModelConfig
from .weights import Tensors


@dataclass
class _Layer:
    spec: LayerSpec
    w_cat: torch.Tensor = None          # attention: [q | k | v | gate]; delta rule: [r | k | v | gate | a | w1]
    w_o: torch.Tensor = None
    w2: Optional[torch.Tensor] = None   # delta rule: decay low-rank up-projection
    rank: int = 0
    f: Dict[str, torch.Tensor] = field(default_factory=dict)     # small fp32 parameters
    w_up: Optional[torch.Tensor] = None
    w_down: Optional[torch.Tensor] = None


class HybridPiece:
    def __init__(self, cfg: ModelConfig, layers: Iterable[int], first: bool, last: bool, tensors: Tensors,
                 device: torch.device, max_tokens: int, max_seqs: int, num_pages: int, quant: str = "bf16",
                 units: Optional[tuple] = None, dtype: torch.dtype = torch.bfloat16, state_slots: int = 0,
                 max_out_rows: int = 0):
        assert cfg.hybrid, "HybridPiece serves configs with per-layer mixer specs"
        if not (first and last):
            raise ValueError(f"{cfg.name}: recurrent state and residual streams are not handed between GPUs yet; "
                             "hybrid models run as a single piece")
        if quant != "bf16":
            raise ValueError(f"{cfg.name}: quantised weights are not implemented for hybrid models")
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("dtype must be bfloat16 or float32")
        self.cfg, self.layers, self.first, self.last = cfg, list(layers), first, last
        self.device = dev = torch.device(device)
        self.dtype = dtype
        self.max_tokens, self.max_seqs, self.num_pages = max_tokens, max_seqs, num_pages
        self.state_slots = max(1, state_slots or max_seqs)
        self.max_out_rows = max(max_out_rows, max_seqs)
        self.head_mode, self.tail_mode = 0, 2
        self.fp8 = self.mx = self.mx_fuse = self.mx_hand = False
        self.max_splits = 1
        self.ns = max(1, cfg.streams)
        W = cfg.hidden_size
        self.Wp = ops.pad_to(W, 64)
        f32 = torch.float32

        def mat(*names, k_mult=64):          # row-concatenated, padded to the GEMM tile, in the operand dtype
            w = torch.cat([tensors[n].to(device=dev, dtype=f32) for n in names], 0)
            return ops.pad_weight(w, 128, k_mult).to(dtype).contiguous()

        def vec(name):
            return tensors[name].to(device=dev, dtype=f32).contiguous()

        self.L: Dict[int, _Layer] = {}
        for l in self.layers:
            sp, p = cfg.layer_specs[l], f"l{l}."
            L = _Layer(spec=sp)
            if sp.mixer == "attention":
                L.w_cat = mat(p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g")
                for n in ("q.norm", "k.norm", "pb"):
                    L.f[n] = vec(p + "mix." + n)
            else:
                L.rank = tensors[p + "mix.w1"].shape[0]
                L.w_cat = mat(p + "mix.r", p + "mix.k", p + "mix.v", p + "mix.g", p + "mix.a", p + "mix.w1")
                L.w2 = mat(p + "mix.w2")
                for n in ("w0", "a.b", "norm"):
                    L.f[n] = vec(p + "mix." + n)
            L.w_o = mat(p + "mix.o")
            L.f["norm1"] = vec(p + "norm1")
            if sp.ff:
                L.w_up, L.w_down = mat(p + "mlp.up"), mat(p + "mlp.down", k_mult=128)   # K of down = padded rows of up
                L.f["norm2"] = vec(p + "norm2")
            if cfg.streams:
                for q in ("hc1", "hc2") if sp.ff else ("hc1",):
                    for n in ("in", "out", "mix"):
                        L.f[f"{q}.{n}"] = vec(f"{p}{q}.{n}")
            self.L[l] = L
        self.embed = tensors["embed"].to(device=dev, dtype=dtype).contiguous()
        self.pair = tensors["bigram"].to(device=dev, dtype=dtype).contiguous() if cfg.pair_buckets else None
        self.final_norm = vec("final.norm")
        self.w_head = mat("head")
        self.vocab_pad = self.w_head.shape[0]

        # ---- per-sequence state (indexed by batch slot) and the paged KV cache of the attention layers
        self.prev_tok = torch.zeros(self.state_slots, device=dev, dtype=torch.int32)
        self.state: Dict[int, torch.Tensor] = {}
        self.k_cache: Dict[int, torch.Tensor] = {}
        self.v_cache: Dict[int, torch.Tensor] = {}
        for l in self.layers:
            sp = cfg.layer_specs[l]
            if sp.mixer == "attention":
                self.k_cache[l] = torch.zeros((num_pages, ops.PAGE, sp.kv_heads, sp.dim), device=dev, dtype=dtype)
                self.v_cache[l] = torch.zeros((num_pages, ops.PAGE, sp.kv_heads, sp.vdim), device=dev, dtype=dtype)
            else:
                self.state[l] = torch.zeros((self.state_slots, sp.heads, sp.dim, sp.dim), device=dev, dtype=f32)
        # ---- activations (every buffer is keyed by its logical width so zero padding is never dirtied)
        self.streams = torch.zeros((max_tokens, self.ns, W), device=dev, dtype=f32)
        self._bufs: Dict[tuple, torch.Tensor] = {}
        self.h = self._buf("h", dtype, self.Wp)
        self.last_x = torch.zeros((self.max_out_rows, self.Wp), device=dev, dtype=dtype)
        self.logits = torch.zeros((self.max_out_rows, self.vocab_pad), device=dev, dtype=f32)
        self._ones = torch.ones(self.ns, device=dev, dtype=f32)
        self.debug_layers: Optional[list] = None     # tests: set to [] to collect the stream sum after every layer

    # ------------------------------------------------------------------ helpers
    def _buf(self, tag: str, dtype: torch.dtype, width: int) -> torch.Tensor:
        key = (tag, dtype, width)
        b = self._bufs.get(key)
        if b is None:
            b = self._bufs[key] = torch.zeros((self.max_tokens, width), device=self.device, dtype=dtype)
        return b

    def weight_bytes(self) -> int:
        n = sum(t.numel() * t.element_size() for L in self.L.values()
                for t in (L.w_cat, L.w_o, L.w2, L.w_up, L.w_down) if t is not None)
        n += self.w_head.numel() * self.w_head.element_size() + self.embed.numel() * self.embed.element_size()
        return n + (self.pair.numel() * self.pair.element_size() if self.pair is not None else 0)

    def streamed_weight_bytes(self) -> int:
        """bytes a decode step streams: every matrix except the embedding tables (one row per sequence is gathered)"""
        n = sum(t.numel() * t.element_size() for L in self.L.values()
                for t in (L.w_cat, L.w_o, L.w2, L.w_up, L.w_down) if t is not None)
        return n + self.w_head.numel() * self.w_head.element_size()

    def state_bytes_per_seq(self) -> int:
        return sum(s[0].numel() * 4 for s in self.state.values())

    def n_launches(self) -> int:
        n = 3          # embedding, final stream sum + norm, previous-token commit (+ the head GEMM counted by the runner)
        for L in self.L.values():
            n += (5 if L.spec.mixer == "attention" else 7) + (3 if L.spec.ff else 0)
        return n

    # ------------------------------------------------------------------ forward
    def forward(self, m, x_in=None, hand=None, out_x=None, h_in=None) -> torch.Tensor:
        """Runs all layers for the spans described by ``m`` (``native.BatchMeta`` with ``seq_slot``); returns fp32
        logits ``[m.n_out or m.n_seqs, vocab_pad]`` for the token rows ``m.last_idx`` (decode: one row per sequence)."""
        c = self.cfg
        T, S, mq = m.n_tokens, m.n_seqs, m.max_q
        eps, mult = c.norm_eps, c.residual_mult
        st = self.streams[:T]
        seq_slot = m.seq_slot
        assert seq_slot is not None, "hybrid models need BatchMeta.seq_slot (state slot of every sequence)"
        ops.hyb_embed(m.ids, m.positions, m.q_start, m.q_len, seq_slot, self.prev_tok, self.embed, self.pair,
                      c.pair_buckets, c.pair_mul_prev, c.pair_mul_cur, st, S, mq)
        h = self.h[:T]
        pend = None                      # (y, mix, out) of the sublayer whose output has not joined the streams yet

        def pre(pend, L, q):
            kw = {}
            if pend is not None:
                kw = dict(y=pend[0], mix=pend[1], outw=pend[2], mult=mult)
            ops.hc_step(st, m.q_start, m.q_len, S, mq, inw=L.f.get(f"hc{q}.in"), gamma=L.f[f"norm{q}"], eps=eps, h=h, **kw)

        for l in self.layers:
            L = self.L[l]
            pre(pend, L, 1)
            y = self._attention(l, L, h, m) if L.spec.mixer == "attention" else self._delta(l, L, h, m)
            pend = (y, L.f.get("hc1.mix"), L.f.get("hc1.out"))
            if L.spec.ff:
                pre(pend, L, 2)
                hid = self._buf("ff", self.dtype, L.w_up.shape[0])[:T]
                ops.linear(L.w_up, h, hid, act=ops.ACT_RELU_SQ)
                y = ops.linear(L.w_down, hid, self._buf("y", torch.float32, L.w_down.shape[0])[:T])
                pend = (y, L.f.get("hc2.mix"), L.f.get("hc2.out"))
            if self.debug_layers is not None:
                self.debug_layers.append(self._debug_sum(st, pend, T))
        # output rows only: last sublayer joins the streams, streams are summed, model norm
        R = m.n_out or S
        if m.last_idx is not None:
            rows = m.last_idx
        else:
            rows = m.q_start           # decode: one token per sequence, row = q_start
        xl = self.last_x[:R]
        kw = dict(y=pend[0], mix=pend[1], outw=pend[2], mult=mult) if pend is not None else {}
        ops.hc_step(st, m.q_start, m.q_len, S, mq, inw=self._ones, gamma=self.final_norm, eps=eps, h=xl, rows=rows,
                    n_rows=R, **kw)
        ops.hyb_commit_prev(m.ids, m.q_start, m.q_len, seq_slot, self.prev_tok, S)
        return ops.linear(self.w_head, xl, self.logits[:R])

    def _debug_sum(self, st: torch.Tensor, pend, T: int) -> torch.Tensor:
        """sum of the streams after the pending sublayer output has joined them (plain torch, tests only)"""
        W, mult = self.cfg.hidden_size, self.cfg.residual_mult
        y, mix, outw = pend
        mix = mix if mix is not None else torch.ones((1, 1), device=st.device)
        outw = outw if outw is not None else torch.ones(1, device=st.device)
        new = torch.einsum("kj,tkw->tjw", mix, st) + mult * outw[None, :, None] * y[:T, None, :W]
        return new.sum(1).clone()

    def _attention(self, l: int, L: _Layer, h: torch.Tensor, m) -> torch.Tensor:
        sp, c = L.spec, self.cfg
        T = m.n_tokens
        H, G, D, V = sp.heads, sp.kv_heads, sp.dim, sp.vdim
        proj = ops.linear(L.w_cat, h, self._buf("proj", torch.float32, L.w_cat.shape[0])[:T])
        q = self._buf("q", torch.float32, H * D)[:T]
        ops.attn_prep(proj, L.f["q.norm"], L.f["k.norm"], m.slots, q, self.k_cache[l], self.v_cache[l], T, H, G, D, V,
                      c.norm_eps)
        ao = self._buf(f"mix{H * V}", self.dtype, L.w_o.shape[1])[:T]
        ops.sig_attention(q, self.k_cache[l], self.v_cache[l], proj, H * D + G * D + G * V, L.f["pb"], ao, m.block_table,
                          m.q_start, m.q_len, m.kv_len, m.n_seqs, m.max_q, H, G, D, V, sp.chunk, sp.scale)
        return ops.linear(L.w_o, ao, self._buf("y", torch.float32, L.w_o.shape[0])[:T])

    def _delta(self, l: int, L: _Layer, h: torch.Tensor, m) -> torch.Tensor:
        sp, c = L.spec, self.cfg
        T = m.n_tokens
        H, D = sp.heads, sp.dim
        d = H * D
        proj = ops.linear(L.w_cat, h, self._buf("proj", torch.float32, L.w_cat.shape[0])[:T])
        th = self._buf(f"lr{L.rank}", self.dtype, L.w2.shape[1])[:T]
        ops.act_cols(proj, 5 * d, th, L.rank, 1, T)                      # tanh of the low-rank decay projection
        lora = ops.linear(L.w2, th, self._buf("lora", torch.float32, L.w2.shape[0])[:T])
        o = self._buf("o", torch.float32, d)[:T]
        ops.delta_scan(proj, 0, d, 2 * d, 4 * d, lora, L.f["w0"], L.f["a.b"], self.state[l], o, m.q_start, m.q_len,
                       m.kv_len, m.seq_slot, m.n_seqs, m.max_q, H, D, D)
        do = self._buf(f"mix{d}", self.dtype, L.w_o.shape[1])[:T]
        ops.delta_post(o, proj, 3 * d, L.f["norm"], do, T, H, D, c.norm_eps)
        return ops.linear(L.w_o, do, self._buf("y", torch.float32, L.w_o.shape[0])[:T])
